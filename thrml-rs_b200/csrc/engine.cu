// Host side of the device library libthrml_b200: context, program upload, chain state, launches of the block-update
// and observer kernels (update_kernels.cuh, observer_kernels.cuh, dense.cuh) and the sweep / schedule drivers.
// sm_100a only; there is no CPU path in this file — without a CUDA device every entry point returns THRML_ERR_CUDA.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <memory>

#include "comm.h"
#include "ctx.h"
#include "dense.cuh"
#include "devbuf.h"
#include "device_math.cuh"
#include "observer_kernels.cuh"
#include "tables.h"
#include "update_kernels.cuh"

using namespace thrml;

struct BlockProg {
    int32_t kind = 0;     // 0 spin, K categorical
    int32_t sd = 0;       // class index
    int32_t is_cat = 0;
    int64_t n = 0, offset = 0;
    int32_t kernel = 0;   // 0 generic spin, 1 threshold table, 2 categorical
    int32_t n_tabs = 0;
    std::vector<std::unique_ptr<DevBuf>> bufs;  // idx/active/w storage
    std::vector<DevTable> host_tabs;
    std::vector<DevBuf*> w_bufs;                // per table, for update_weights
    std::vector<size_t> w_len;
    std::vector<DevBuf*> rows_bufs;             // per table: int32 [n*k], the row of the source group each slot copies (program.rs:216-235)
    std::vector<int32_t> src_group, tab_wdim;   // per table: index of the source interaction group, weights per slot
    DevBuf d_tabs;   // DevTable[n_tabs]
    DevBuf d_nbr;    // int32 [n][8] (threshold-table kernel)
    DevBuf d_lut;    // uint32 [n][256]
    DevBuf d_seq_nbr, d_seq_w, d_seq_first, d_seq_cnt;  // entry lists of the sequential-sum kernel (kernels 4 and 6)
    DevBuf d_seq_overflow, d_seq_n_rows;                 // kernels 4 and 6: overflow rows of nodes with more than 32 entries
    int64_t seq_rows = 0;
    std::vector<char> h_hub;                             // kernels 4 and 6: nodes with overflow rows (not served by the fused observer)
    DevBuf d_seq_order, d_seq_counter;                   // kernels 4 and 6: nodes by decreasing entry count; the launch's work counter
    DevBuf d_split_row, d_split_nodes, d_split_tab, d_split_margin;  // kernels 4 and 6: split field tables of the nodes with one entry row
    int64_t n_split = 0;
    bool split_wide = false;  // some node has four tables
    DevBuf d_wide_ent, d_wide_first, d_wide_cnt;         // kernel 7: entry lists (table and slot) of the wide general spin kernel
    bool wide_has_cat = false;                           // kernel 7: some table has a categorical tail
    int32_t cat_most = 0;                                // kernels 5 and 8: largest active slot count of a node
    bool cat_warp = false;                               // kernel 5: entry lists (d_wide_*) exist for the warp-per-node categorical kernel
    DevBuf d_lut_row, d_lut_nodes;                       // kernel 6: table row of each node (-1 = sequential-sum node) and its inverse
    int64_t n_lut = 0;                                   // kernel 6: nodes that have a threshold table
    std::vector<int32_t> h_nbr;  // host copy of d_nbr
    int32_t max_deg = 0;         // largest number of neighbour slots any node of the block uses (threshold-table blocks)
    int32_t order = -1;          // position of the block's superblock in the sweep; -1 for clamped blocks
    // dense bipartite path (kernel 3): every neighbour of every node lies in block `dense_src`
    int32_t dense_src = -1;      // candidate source block, -1 when the block does not qualify
    bool dense_on = false;
    int32_t base_kernel = 0;     // kernel used when the dense path is off or cannot serve a call
    int64_t dense_pitch = 0;     // elements per row of d_dense_w
    int32_t dense_bn = 128;      // tile width of the update GEMM
    int32_t dense_bn_pair = 128; // tile width when CTA pairs share 256-row tiles
    std::vector<float> h_dense_w;  // [n][n_src] f32, canonical weights (0 where there is no edge)
    std::vector<float> h_dense_bias;
    DevBuf d_dense_w;            // bf16 [n][dense_pitch], K-major (K = source nodes)
    DevBuf d_dense_bias;         // f32 [n]
    CUtensorMap map_w;
    CUtensorMap map_w_pair;      // same operand, box of dense_bn_pair / 2 rows
};

struct thrml_program {
    thrml_ctx* ctx = nullptr;
    int device = 0;
    int32_t n_free = 0, n_clamped = 0, n_classes = 0, sd_spin = -1, sd_cat = -1;
    std::vector<int64_t> class_size;
    std::vector<BlockProg> blocks;  // free ++ clamped
    std::vector<std::vector<int32_t>> sampling_order;
    std::vector<uint8_t> staged;    // per superblock: 1 when its blocks read positions the superblock itself writes
    int64_t max_stage_rows = 0;
    std::vector<int8_t> loc_sd;     // node -> class / position (host copy, for observers)
    std::vector<int64_t> loc_pos;
    std::vector<uint8_t> is_dense_source;  // per block: some dense block reads its +-1 image
    bool any_dense = false;
    int32_t kernel_epoch = 0;  // bumped whenever a block changes kernel; observers built before that stop fusing
    int32_t dense_tiles = 2;         // THRML_OPT_DENSE_TILES
    float split_extra_margin = 0.f;  // THRML_OPT_SPLIT_MARGIN
    bool gather_only = false;        // THRML_OPT_GATHER_ONLY
    int32_t state_format = 0;        // THRML_OPT_STATE_FORMAT: 1 = sweeps of all-threshold-table programs run on a bit-packed mirror
};

struct thrml_state {
    thrml_program* prog = nullptr;
    int device = 0;
    int64_t n_chains = 0, chain_offset = 0, ld = 0;
    DevBuf cls[2];      // state rows per class
    DevBuf stage;       // staging rows for superblocks that cannot be updated in place
    DevBuf scratch;     // transposes, injected noise, debug fields
    // dense path: +-1 bf16 image [chain][node] of source blocks, tensor maps, per-row one counts, error flag
    std::vector<std::unique_ptr<DevBuf>> image;
    std::vector<uint8_t> image_fresh, ones_fresh;
    std::vector<CUtensorMap> map_image;
    std::vector<std::unique_ptr<DevBuf>> ones;
    DevBuf d_err, d_corr, d_dense_debug;
    // sweeps queued for the persistent kernel (cache-resident programs): (sweep key, observer to accumulate or null)
    std::vector<std::pair<uint64_t, thrml_moments*>> pending;
    DevBuf d_plan, d_plan_acc, d_slice_blocks;
    int persist_grid = 0;  // CTAs of the persistent kernel (all co-resident), 0 = not eligible
    int32_t no_image_block = -1;  // a dense update of this block skips its +-1 image (nobody reads it before the next update)
    bool sliced = false;   // the chain-sliced kernel serves the queue instead (four chains of every spin fit in shared memory)
    int64_t persist_epoch = -1;  // program kernel_epoch persist_grid was computed for
    int64_t persistent_launches = 0, block_launches = 0;
    int64_t image_rows = 0;
    // Bit-packed mirror of the spin class (THRML_OPT_STATE_FORMAT = 1): uint32 [position][pw], chain c at bit c & 31 of word
    // c >> 5.  At most one of the two copies is stale; every access to either goes through rows() / packed_rows(), which
    // make the requested copy current first and assume the caller will write it.
    mutable DevBuf packed;
    int64_t pw = 0;
    mutable bool bytes_valid = true, packed_valid = false;
    void touch(int32_t block) { if (!image_fresh.empty()) { image_fresh[block] = 0; ones_fresh[block] = 0; } }
    uint8_t* rows(int sd) const {
        if (packed.p && sd == prog->sd_spin) {
            if (!bytes_valid) {
                const int64_t n_rows = prog->class_size[sd], units = n_rows * (ld >> 4);
                k_unpack_rows<<<static_cast<unsigned>((units + 255) / 256), 256, 0, prog->ctx->stream>>>(packed.as<uint32_t>(), pw, n_rows, ld, n_chains, cls[sd].as<uint8_t>());
                bytes_valid = true;
            }
            packed_valid = false;
        }
        return cls[sd].as<uint8_t>();
    }
    int32_t packed_rows(uint32_t** out) {
        const int sd = prog->sd_spin;
        const int64_t n_rows = prog->class_size[sd];
        if (!packed.p) {
            pw = (ld + 31) / 32;
            if (int32_t rc = packed.alloc(static_cast<size_t>(n_rows) * pw * 4)) return rc;
            packed_valid = false;
        }
        if (!packed_valid) {
            k_pack_rows<<<static_cast<unsigned>((n_rows + 7) / 8), dim3(32, 8), 0, prog->ctx->stream>>>(cls[sd].as<uint8_t>(), ld, n_chains, n_rows, pw, packed.as<uint32_t>());
            packed_valid = true;
        }
        bytes_valid = false;
        *out = packed.as<uint32_t>();
        return THRML_OK;
    }
};

struct FusedMaps {
    DevBuf m1;  // int32 [n]: row of <s_i>, -1 when not accumulated by the block's update kernel
    DevBuf m2;  // int32 [n][8]: row of <s_i s_j> per neighbour slot, -1 when not owned by this node
};

struct thrml_moments {
    thrml_program* prog = nullptr;
    int device = 0;
    // rows the threshold-table kernels accumulate while they update (per free block), and the rest
    std::vector<std::unique_ptr<FusedMaps>> fused;
    bool any_fused = false;
    int32_t kernel_epoch = 0;  // program epoch the fused maps were built for
    int64_t n_left = 0;
    DevBuf d_left_ptr, d_left_sd, d_left_pos, d_left_rows;
    int32_t mode = 0;  // 0 products over tuples, 1 per-node category counts
    int32_t spin_transform = 1;
    std::vector<int64_t> rows_per_type;
    int64_t total_rows = 0;
    int32_t K = 0;
    DevBuf d_row_ptr, d_mem_sd, d_mem_pos;  // mode 0: CSR of members (class, position)
    bool all_spin = false, left_all_spin = false;  // every member of every (left-over) row is a spin read as +-1: the XOR kernel serves them
    DevBuf d_node_sd, d_node_pos;           // mode 1: observed nodes
    DevBuf d_sums;                          // int64 [total_rows] (mode 0) or [nodes*K] (mode 1), then two spare slots for the allreduce
    DevBuf d_narrow;                        // int32 copy of the sums for the allreduce when every total fits 32 bits
    int64_t n_obs = 0;
    int64_t sum_slots() const { return std::max<int64_t>(total_rows, 1); }
};

// ---------------------------------------------------------------------------------------------------------
// Host helpers.
// ---------------------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}
// 2-D K-major operand: `rows` rows of `k_elems` contiguous elements, row pitch in bytes; box = 128 bytes of K x box_rows,
// 128-byte swizzle, out-of-range elements read as zero.
static int32_t make_operand_map(CUtensorMap* map, void* base, bool is_u8, int64_t k_elems, int64_t rows, int64_t pitch_bytes, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(THRML_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k_elems), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_bytes)};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(is_u8 ? 128 : 64), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, is_u8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(THRML_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
    return THRML_OK;
}
// Width of a CTA pair's tile for n output columns: the candidate that pads n the least, the wider one on ties.
static int32_t pair_tile_width(int64_t n) {
    int32_t best = 256;
    for (int32_t w : {208, 128})
        if ((n + w - 1) / w * w < (n + best - 1) / best * best) best = w;
    return best;
}
// 0 = one CTA per 128-row tile, 1 = CTA pairs on 256-row tiles, 2 = per launch, whichever suits the shape: pairs halve the
// B-operand traffic per SM, which pays when the GEMM is bound by its operand feed (long K); a short-K update is bound
// by its sampling epilogue and runs a little faster without the cluster hand-overs.
static bool use_pair_tiles(int32_t mode, int64_t m_rows, int64_t k_elems) {
    if (mode != 2) return mode == 1;
    const int64_t pad_pair = (m_rows + 255) / 256 * 256, pad_single = (m_rows + 127) / 128 * 128;
    return k_elems >= 2048 && pad_pair * 10 <= pad_single * 11;
}
static inline uint16_t f32_to_bf16_rn(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    u += 0x7fffu + ((u >> 16) & 1u);
    return static_cast<uint16_t>(u >> 16);
}
static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = static_cast<uint32_t>(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
static int32_t upload(DevBuf& buf, const void* host, size_t bytes, cudaStream_t st) {
    if (int32_t rc = buf.alloc(bytes)) return rc;
    if (bytes) CU_TRY(cudaMemcpyAsync(buf.p, host, bytes, cudaMemcpyHostToDevice, st));
    return THRML_OK;
}
// Launch shape of the kernels whose thread is one node x four chains: 256 threads as (chain quads, nodes).  With 128 chains
// or more a warp spans 32 quads of one node; with fewer the block is narrower and a warp covers several nodes, so a
// single-chain state (the reference's usual call) does not idle 31 lanes of 32.
static dim3 block_nq(int64_t ld) {
    unsigned qx = 1;
    while (qx < 32 && static_cast<int64_t>(qx) * 4 < ld) qx *= 2;
    return dim3(qx, 256 / qx);
}
static dim3 grid_nq(int64_t n, int64_t ld) {
    const dim3 b = block_nq(ld);
    return dim3(static_cast<unsigned>((n + b.y - 1) / b.y), static_cast<unsigned>((ld / 4 + b.x - 1) / b.x));
}
static int32_t need_scratch(thrml_state* s, size_t bytes) {
    if (s->scratch.holds(bytes)) return THRML_OK;
    CU_TRY(cudaStreamSynchronize(s->prog->ctx->stream));
    return s->scratch.alloc(bytes);
}

extern "C" {

int32_t thrml_ctx_create(int32_t device_id, thrml_ctx** out) {
    if (!out) return fail(THRML_ERR_INVALID_ARG, "null output");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) return fail(THRML_ERR_CUDA, std::string("no usable CUDA device: ") + cudaGetErrorString(e));
    if (device_id < 0 || device_id >= count) return fail(THRML_ERR_INVALID_ARG, "device id out of range");
    CU_TRY(cudaSetDevice(device_id));
    auto ctx = std::make_unique<thrml_ctx>();
    ctx->device = device_id;
    CU_TRY(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
    cudaDeviceProp prop;
    CU_TRY(cudaGetDeviceProperties(&prop, device_id));
    ctx->sm_count = prop.multiProcessorCount;
    *out = ctx.release();
    return THRML_OK;
}
void thrml_ctx_destroy(thrml_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}
int32_t thrml_ctx_synchronize(thrml_ctx* ctx) {
    if (!ctx) return fail(THRML_ERR_INVALID_ARG, "null context");
    CU_TRY(cudaStreamSynchronize(ctx->stream));
    return THRML_OK;
}
void* thrml_ctx_stream(thrml_ctx* ctx) { return ctx ? static_cast<void*>(ctx->stream) : nullptr; }

// ---------------------------------------------------------------------------------------------------------
// Program.
// ---------------------------------------------------------------------------------------------------------
static int32_t rebuild_seq(thrml_program* p, BlockProg& bp) {
    k_build_seq<<<static_cast<unsigned>((bp.n + 255) / 256), 256, 0, p->ctx->stream>>>(bp.d_tabs.as<DevTable>(), bp.n_tabs, static_cast<int32_t>(bp.n),
                                                                                      bp.d_seq_overflow.as<int32_t>(), bp.d_seq_nbr.as<int32_t>(),
                                                                                      bp.d_seq_w.as<float>(), bp.d_seq_first.as<uint32_t>(), bp.d_seq_cnt.as<int32_t>());
    CU_TRY(cudaGetLastError());
    if (bp.n_split > 0) {
        k_build_split<<<static_cast<unsigned>(bp.n_split), 256, 0, p->ctx->stream>>>(bp.d_split_nodes.as<int32_t>(), bp.d_split_row.as<int32_t>(), bp.d_seq_nbr.as<int32_t>(), bp.d_seq_w.as<float>(),
                                                                                    bp.d_seq_cnt.as<int32_t>(), bp.d_split_tab.as<float>(), bp.d_split_margin.as<float>(), p->split_extra_margin);
        CU_TRY(cudaGetLastError());
    }
    return THRML_OK;
}
static int32_t rebuild_lut(thrml_program* p, BlockProg& bp) {
    const int64_t rows = bp.base_kernel == 6 || bp.kernel == 6 ? bp.n_lut : bp.n;  // a mixed block keeps tables for some of its nodes only
    const int64_t total = rows * LUT_SIZE;
    if (total == 0) return THRML_OK;
    k_build_lut<<<static_cast<unsigned>((total + 255) / 256), 256, 0, p->ctx->stream>>>(bp.d_tabs.as<DevTable>(), bp.n_tabs, static_cast<int32_t>(rows),
                                                                                         bp.d_lut.as<uint32_t>(), bp.d_lut_nodes.p ? bp.d_lut_nodes.as<int32_t>() : nullptr);
    CU_TRY(cudaGetLastError());
    return THRML_OK;
}

int32_t thrml_program_create(thrml_ctx* ctx, const thrml_builder* b, thrml_program** out) {
    if (!ctx || !b || !out) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (!b->compiled) return fail(THRML_ERR_INVALID_ARG, "builder is not compiled");
    CU_TRY(cudaSetDevice(ctx->device));
    auto p = std::make_unique<thrml_program>();
    p->ctx = ctx;
    p->device = ctx->device;
    p->n_free = static_cast<int32_t>(b->free_blocks.size());
    p->n_clamped = static_cast<int32_t>(b->clamped_blocks.size());
    p->n_classes = b->n_classes;
    p->sd_spin = b->sd_spin;
    p->sd_cat = b->sd_cat;
    p->class_size = b->class_size;
    p->sampling_order = b->sampling_order;
    p->loc_sd = b->loc_sd;
    p->loc_pos = b->loc_pos;
    p->blocks.resize(p->n_free + p->n_clamped);
    for (int32_t i = 0; i < p->n_free + p->n_clamped; ++i) {
        const BlockInfo& bi = i < p->n_free ? b->free_blocks[i] : b->clamped_blocks[i - p->n_free];
        BlockProg& bp = p->blocks[i];
        bp.kind = bi.kind;
        bp.sd = bi.sd;
        bp.is_cat = bi.kind != 0;
        bp.n = static_cast<int64_t>(bi.nodes.size());
        bp.offset = bi.offset;
        if (i >= p->n_free) continue;
        // SoftmaxConditional (softmax.rs:147-222) keeps only the tables with one weight per category and never reads a
        // neighbour: its block runs the categorical kernels on those tables with their tails dropped.
        std::vector<SlotTable> softmax_tabs;
        if (bi.sampler == THRML_SAMPLER_SOFTMAX) {
            for (const SlotTable& t : b->tables[i]) {
                if (t.wdim != bi.kind) continue;
                SlotTable c = t;
                c.idx.clear();
                c.tail_sd.clear();
                c.tail_is_cat.clear();
                c.n_spin = 0;
                softmax_tabs.push_back(std::move(c));
            }
        }
        const auto& tabs = bi.sampler == THRML_SAMPLER_SOFTMAX ? softmax_tabs : b->tables[i];
        bp.n_tabs = static_cast<int32_t>(tabs.size());
        bp.kernel = bp.is_cat ? 2 : 0;
        bool lut_ok = !bp.is_cat && !tabs.empty();
        for (const SlotTable& t : tabs) {
            const int32_t n_tails = static_cast<int32_t>(t.idx.size());
            if (n_tails > MAX_TAILS) return fail(THRML_ERR_UNSUPPORTED, "an interaction group has more than 8 tail node blocks");
            if (n_tails - t.n_spin > 1) return fail(THRML_ERR_UNSUPPORTED, "only the first categorical tail of a group is honoured by the reference samplers; groups with two or more are not supported");
            const bool has_cat = n_tails > t.n_spin;
            if (bp.is_cat) {
                if (t.wdim != (has_cat ? bp.kind * bp.kind : bp.kind))
                    return fail(THRML_ERR_UNSUPPORTED, "categorical block weights must be [rows, K, 1] or [rows, K, K] with K the block's category count");
            } else if (!has_cat && t.wdim != 1) {
                return fail(THRML_ERR_UNSUPPORTED, "spin block weights without a categorical tail must be [rows, 1, 1]");
            }
            if (has_cat || t.wdim != 1 || n_tails != t.n_spin || t.n_spin > 1) lut_ok = false;
            DevTable d{};
            d.k = t.k; d.wdim = t.wdim; d.n_spin = t.n_spin; d.n_tails = n_tails;
            for (int32_t tl = 0; tl < n_tails; ++tl) {
                bp.bufs.emplace_back(new DevBuf());
                if (int32_t rc = upload(*bp.bufs.back(), t.idx[tl].data(), t.idx[tl].size() * 4, ctx->stream)) return rc;
                d.idx[tl] = bp.bufs.back()->as<int32_t>();
            }
            bp.bufs.emplace_back(new DevBuf());
            if (int32_t rc = upload(*bp.bufs.back(), t.active.data(), t.active.size(), ctx->stream)) return rc;
            d.active = bp.bufs.back()->as<uint8_t>();
            bp.bufs.emplace_back(new DevBuf());
            if (int32_t rc = upload(*bp.bufs.back(), t.w.data(), t.w.size() * 4, ctx->stream)) return rc;
            d.w = bp.bufs.back()->as<float>();
            bp.w_bufs.push_back(bp.bufs.back().get());
            bp.w_len.push_back(t.w.size());
            bp.bufs.emplace_back(new DevBuf());
            if (int32_t rc = upload(*bp.bufs.back(), t.rows.data(), t.rows.size() * 4, ctx->stream)) return rc;
            bp.rows_bufs.push_back(bp.bufs.back().get());
            bp.src_group.push_back(t.source_group);
            bp.tab_wdim.push_back(t.wdim);
            bp.host_tabs.push_back(d);
        }
        if (int32_t rc = upload(bp.d_tabs, bp.host_tabs.data(), bp.host_tabs.size() * sizeof(DevTable), ctx->stream)) return rc;
        const bool single_spin_tails = lut_ok;  // every table: scalar weights, no tail or one spin tail
        if (lut_ok) {
            // compact neighbour list in table order, slot order; a node with more than 8 neighbour slots rules the kernel out
            std::vector<int32_t> nbr(static_cast<size_t>(bp.n) * LUT_BITS, -1);
            for (int64_t i2 = 0; i2 < bp.n && lut_ok; ++i2) {
                int cnt = 0;
                for (const SlotTable& t : tabs) {
                    if (t.n_spin != 1) continue;
                    for (int32_t j = 0; j < t.k; ++j) {
                        const size_t flat = static_cast<size_t>(i2) * t.k + j;
                        if (!t.active[flat]) continue;
                        if (cnt == LUT_BITS) { lut_ok = false; break; }
                        nbr[static_cast<size_t>(i2) * LUT_BITS + cnt++] = t.idx[0][flat];
                    }
                    if (!lut_ok) break;
                }
                bp.max_deg = std::max(bp.max_deg, cnt);
            }
            if (lut_ok) {
                if (int32_t rc = upload(bp.d_nbr, nbr.data(), nbr.size() * 4, ctx->stream)) return rc;
                bp.h_nbr = nbr;
                if (int32_t rc = bp.d_lut.alloc(static_cast<size_t>(bp.n) * LUT_SIZE * 4)) return rc;
                if (int32_t rc = rebuild_lut(p.get(), bp)) return rc;
                bp.kernel = 1;
            }
        }
        if (single_spin_tails && bp.kernel == 0) {
            // too many neighbour slots for a threshold table: the sequential-sum kernel, SEQ_MAX entries per row; a node with
            // more entries continues in overflow rows (and leaves the fused observer to the separate kernel)
            std::vector<int32_t> overflow(static_cast<size_t>(bp.n), -1), n_rows(static_cast<size_t>(bp.n), 1);
            int64_t rows = bp.n;
            bp.h_hub.assign(static_cast<size_t>(bp.n), 0);
            for (int64_t i2 = 0; i2 < bp.n; ++i2) {
                int64_t cnt = 0;
                for (const SlotTable& t : tabs)
                    for (int32_t j = 0; j < t.k; ++j) cnt += t.active[static_cast<size_t>(i2) * t.k + j] ? 1 : 0;
                if (cnt > SEQ_MAX) {
                    const int64_t extra = (cnt - 1) / SEQ_MAX;
                    overflow[i2] = static_cast<int32_t>(rows);
                    n_rows[i2] = static_cast<int32_t>(1 + extra);
                    rows += extra;
                    bp.h_hub[i2] = 1;
                }
            }
            if (rows < (int64_t(1) << 26)) {
                bp.h_nbr.assign(static_cast<size_t>(bp.n) * SEQ_MAX, -1);  // the entry order of k_build_seq (first row of each node)
                for (int64_t i2 = 0; i2 < bp.n; ++i2) {
                    int e = 0;
                    for (const SlotTable& t : tabs)
                        for (int32_t j = 0; j < t.k; ++j) {
                            const size_t flat = static_cast<size_t>(i2) * t.k + j;
                            if (!t.active[flat]) continue;
                            if (t.n_spin == 1 && e < SEQ_MAX) bp.h_nbr[static_cast<size_t>(i2) * SEQ_MAX + e] = t.idx[0][flat];
                            ++e;
                        }
                }
                bp.seq_rows = rows;
                if (int32_t rc = bp.d_seq_nbr.alloc(static_cast<size_t>(rows) * SEQ_MAX * 4)) return rc;
                if (int32_t rc = bp.d_seq_w.alloc(static_cast<size_t>(rows) * SEQ_MAX * 4)) return rc;
                if (int32_t rc = bp.d_seq_first.alloc(static_cast<size_t>(rows) * 4)) return rc;
                if (int32_t rc = bp.d_seq_cnt.alloc(static_cast<size_t>(rows) * 4)) return rc;
                if (int32_t rc = upload(bp.d_seq_overflow, overflow.data(), overflow.size() * 4, ctx->stream)) return rc;
                if (int32_t rc = upload(bp.d_seq_n_rows, n_rows.data(), n_rows.size() * 4, ctx->stream)) return rc;
                if (int32_t rc = rebuild_seq(p.get(), bp)) return rc;
                {
                    std::vector<int32_t> cnt_of(static_cast<size_t>(bp.n), 0), order(static_cast<size_t>(bp.n));
                    for (int64_t i2 = 0; i2 < bp.n; ++i2) {
                        for (const SlotTable& t : tabs)
                            for (int32_t j = 0; j < t.k; ++j) cnt_of[i2] += t.active[static_cast<size_t>(i2) * t.k + j] ? 1 : 0;
                        order[i2] = static_cast<int32_t>(i2);
                    }
                    std::stable_sort(order.begin(), order.end(), [&](int32_t x, int32_t y) { return cnt_of[x] > cnt_of[y]; });
                    if (int32_t rc = upload(bp.d_seq_order, order.data(), order.size() * 4, ctx->stream)) return rc;
                    if (int32_t rc = bp.d_seq_counter.alloc(4)) return rc;
                }
                bp.kernel = 4;
                // nodes with at most 8 neighbour slots can keep a threshold table: worth a mixed block when they are many
                std::vector<int32_t> lut_row(static_cast<size_t>(bp.n), -1), lut_nodes, nbr8;
                for (int64_t i2 = 0; i2 < bp.n; ++i2) {
                    int deg = 0;
                    for (int e = 0; e < SEQ_MAX; ++e) deg += bp.h_nbr[static_cast<size_t>(i2) * SEQ_MAX + e] >= 0 ? 1 : 0;
                    if (deg > LUT_BITS || bp.h_hub[i2]) continue;
                    lut_row[i2] = static_cast<int32_t>(lut_nodes.size());
                    lut_nodes.push_back(static_cast<int32_t>(i2));
                    int at = 0;
                    int32_t row8[LUT_BITS];
                    for (int e = 0; e < LUT_BITS; ++e) row8[e] = -1;
                    for (int e = 0; e < SEQ_MAX; ++e)
                        if (bp.h_nbr[static_cast<size_t>(i2) * SEQ_MAX + e] >= 0) row8[at++] = bp.h_nbr[static_cast<size_t>(i2) * SEQ_MAX + e];
                    nbr8.insert(nbr8.end(), row8, row8 + LUT_BITS);
                    // the observer indexes a table node's pair rows by neighbour slot: the first 8 entries of its row
                    for (int e = 0; e < SEQ_MAX; ++e) bp.h_nbr[static_cast<size_t>(i2) * SEQ_MAX + e] = e < LUT_BITS ? row8[e] : -1;
                }
                if (static_cast<int64_t>(lut_nodes.size()) * 4 >= bp.n) {
                    bp.n_lut = static_cast<int64_t>(lut_nodes.size());
                    if (int32_t rc = upload(bp.d_lut_row, lut_row.data(), lut_row.size() * 4, ctx->stream)) return rc;
                    if (int32_t rc = upload(bp.d_lut_nodes, lut_nodes.data(), lut_nodes.size() * 4, ctx->stream)) return rc;
                    if (int32_t rc = upload(bp.d_nbr, nbr8.data(), nbr8.size() * 4, ctx->stream)) return rc;
                    if (int32_t rc = bp.d_lut.alloc(static_cast<size_t>(bp.n_lut) * LUT_SIZE * 4)) return rc;
                    bp.kernel = 6;
                    if (int32_t rc = rebuild_lut(p.get(), bp)) return rc;
                } else {
                    // keep the entry order for the observer
                    for (int64_t i2 = 0; i2 < bp.n; ++i2) {
                        int e = 0;
                        for (const SlotTable& t : tabs)
                            for (int32_t j = 0; j < t.k; ++j) {
                                const size_t flat = static_cast<size_t>(i2) * t.k + j;
                                if (!t.active[flat]) continue;
                                if (e < SEQ_MAX) bp.h_nbr[static_cast<size_t>(i2) * SEQ_MAX + e] = t.n_spin == 1 ? t.idx[0][flat] : -1;
                                ++e;
                            }
                    }
                }
                // sequential-sum nodes with one entry row look their field up in two (at most 16 neighbours) or four tables
                {
                    std::vector<int32_t> split_row(static_cast<size_t>(bp.n), -1), split_nodes;
                    int64_t tables = 0;
                    for (int64_t i2 = 0; i2 < bp.n; ++i2) {
                        if (bp.h_hub[i2] || (bp.kernel == 6 && lut_row[i2] >= 0)) continue;
                        int deg = 0;
                        for (int e = 0; e < SEQ_MAX; ++e) deg += bp.h_nbr[static_cast<size_t>(i2) * SEQ_MAX + e] >= 0 ? 1 : 0;
                        if (deg > SPLIT_BITS || tables + 4 >= (int64_t(1) << 30)) continue;
                        const int groups = deg > 16 ? 4 : 2;
                        split_row[i2] = static_cast<int32_t>(2 * tables + (groups == 4 ? 1 : 0));
                        split_nodes.push_back(static_cast<int32_t>(i2));
                        tables += groups;
                        if (groups == 4) bp.split_wide = true;
                    }
                    if (!split_nodes.empty() && static_cast<size_t>(tables) * 1024 <= (size_t(8) << 30)) {
                        bp.n_split = static_cast<int64_t>(split_nodes.size());
                        if (int32_t rc = upload(bp.d_split_row, split_row.data(), split_row.size() * 4, ctx->stream)) return rc;
                        if (int32_t rc = upload(bp.d_split_nodes, split_nodes.data(), split_nodes.size() * 4, ctx->stream)) return rc;
                        if (int32_t rc = bp.d_split_tab.alloc(static_cast<size_t>(tables) * 1024)) return rc;
                        if (int32_t rc = bp.d_split_margin.alloc(static_cast<size_t>(bp.n) * 4)) return rc;
                        if (int32_t rc = rebuild_seq(p.get(), bp)) return rc;
                    }
                }
            }
        }
        if (!bp.is_cat && bp.kernel == 0 && !tabs.empty() && tabs.size() <= 127) {
            // spin block with multi-spin or categorical tails: the warp-per-node general kernel (kind 7) when every node has at
            // most SEQ_MAX active slots and no slot multiplies more than WIDE_SPIN_TAILS spins
            bool ok = true;
            for (const SlotTable& t : tabs) ok = ok && t.k < (1 << 24) && t.n_spin <= WIDE_SPIN_TAILS;
            std::vector<int32_t> ent, cnt;
            std::vector<uint32_t> first;
            if (ok) {
                ent.assign(static_cast<size_t>(bp.n) * SEQ_MAX, -1);
                cnt.assign(static_cast<size_t>(bp.n), 0);
                first.assign(static_cast<size_t>(bp.n), 0);
            }
            for (int64_t i2 = 0; i2 < bp.n && ok; ++i2) {
                int e = 0;
                for (size_t ti = 0; ti < tabs.size() && ok; ++ti) {
                    const SlotTable& t = tabs[ti];
                    bool started = false;
                    for (int32_t j = 0; j < t.k; ++j) {
                        if (!t.active[static_cast<size_t>(i2) * t.k + j]) continue;
                        if (e == SEQ_MAX) { ok = false; break; }
                        if (!started) first[i2] |= 1u << e;
                        started = true;
                        ent[static_cast<size_t>(i2) * SEQ_MAX + e++] = static_cast<int32_t>(ti << 24) | j;
                    }
                }
                if (ok) cnt[i2] = e;
            }
            if (ok) {
                if (int32_t rc = upload(bp.d_wide_ent, ent.data(), ent.size() * 4, ctx->stream)) return rc;
                if (int32_t rc = upload(bp.d_wide_first, first.data(), first.size() * 4, ctx->stream)) return rc;
                if (int32_t rc = upload(bp.d_wide_cnt, cnt.data(), cnt.size() * 4, ctx->stream)) return rc;
                for (const SlotTable& t : tabs) bp.wide_has_cat = bp.wide_has_cat || static_cast<int32_t>(t.idx.size()) > t.n_spin;
                bp.kernel = 7;
            }
        }
        if (bp.is_cat && !tabs.empty()) {
            // categorical block with few active slots per node: the register-resident kernel (kind 5) takes the in-kernel-noise updates
            int64_t most = 0;
            for (int64_t i2 = 0; i2 < bp.n; ++i2) {
                int64_t cnt = 0;
                for (const SlotTable& t : tabs)
                    for (int32_t j = 0; j < t.k; ++j) cnt += t.active[static_cast<size_t>(i2) * t.k + j] ? 1 : 0;
                most = std::max(most, cnt);
            }
            if (most <= CAT_SLOTS) bp.kernel = 5;
            bp.cat_most = static_cast<int32_t>(std::min<int64_t>(most, CAT_MANY_SLOTS));
            // entry lists for the warp-per-node forms (K <= 16, at most three spin tails per slot): kind 5 with up to 8 slots
            // per node keeps them in registers, kind 8 with up to 32 in shared memory
            bool ok = bp.kind <= 16 && tabs.size() <= 127 && most <= CAT_MANY_SLOTS;
            for (const SlotTable& t : tabs) ok = ok && t.k < (1 << 24) && t.n_spin <= WIDE_SPIN_TAILS;
            if (ok && bp.kernel != 5) bp.kernel = 8;
            const int64_t ENT = bp.kernel == 8 ? CAT_MANY_SLOTS : CAT_SLOTS;
            if (ok) {
                std::vector<int32_t> ent(static_cast<size_t>(bp.n) * ENT, -1), cnt(static_cast<size_t>(bp.n), 0);
                std::vector<uint32_t> first(static_cast<size_t>(bp.n), 0);
                for (int64_t i2 = 0; i2 < bp.n; ++i2) {
                    int e = 0;
                    for (size_t ti = 0; ti < tabs.size(); ++ti) {
                        const SlotTable& t = tabs[ti];
                        bool started = false;
                        for (int32_t j = 0; j < t.k; ++j) {
                            if (!t.active[static_cast<size_t>(i2) * t.k + j]) continue;
                            if (!started) first[i2] |= 1u << e;
                            started = true;
                            ent[static_cast<size_t>(i2) * ENT + e++] = static_cast<int32_t>(ti << 24) | j;
                        }
                    }
                    cnt[i2] = e;
                }
                if (int32_t rc = upload(bp.d_wide_ent, ent.data(), ent.size() * 4, ctx->stream)) return rc;
                if (int32_t rc = upload(bp.d_wide_first, first.data(), first.size() * 4, ctx->stream)) return rc;
                if (int32_t rc = upload(bp.d_wide_cnt, cnt.data(), cnt.size() * 4, ctx->stream)) return rc;
                bp.cat_warp = true;
            }
        }
        bp.base_kernel = bp.kernel;
        // Dense bipartite candidate: a spin block whose neighbours all lie in one other spin block, densely enough
        // that the field is a GEMM against that block's +-1 image.
        if (!bp.is_cat && !tabs.empty()) {
            bool ok = true;
            int64_t lo = INT64_MAX, hi = -1, slots = 0;
            for (const SlotTable& t : tabs) {
                if (t.wdim != 1 || t.idx.size() != static_cast<size_t>(t.n_spin) || t.n_spin > 1) { ok = false; break; }
                if (t.n_spin == 0) continue;
                for (size_t f = 0; f < t.active.size(); ++f)
                    if (t.active[f]) { lo = std::min<int64_t>(lo, t.idx[0][f]); hi = std::max<int64_t>(hi, t.idx[0][f]); ++slots; }
            }
            int32_t src = -1;
            if (ok && hi >= 0)
                for (int32_t o = 0; o < p->n_free + p->n_clamped; ++o) {
                    const BlockInfo& ob = o < p->n_free ? b->free_blocks[o] : b->clamped_blocks[o - p->n_free];
                    if (ob.kind == 0 && o != i && lo >= ob.offset && hi < ob.offset + static_cast<int64_t>(ob.nodes.size())) src = o;
                }
            if (src >= 0) {
                const BlockInfo& ob = src < p->n_free ? b->free_blocks[src] : b->clamped_blocks[src - p->n_free];
                const int64_t n_src = static_cast<int64_t>(ob.nodes.size());
                if (n_src >= 16 && bp.n * n_src <= (int64_t(1) << 28) && 4 * slots >= bp.n * n_src) {
                    bp.dense_src = src;
                    bp.h_dense_w.assign(static_cast<size_t>(bp.n * n_src), 0.0f);
                    bp.h_dense_bias.assign(static_cast<size_t>(bp.n), 0.0f);
                    for (const SlotTable& t : tabs)
                        for (int64_t i2 = 0; i2 < bp.n; ++i2) {
                            float sum = 0.0f;
                            for (int32_t j = 0; j < t.k; ++j) {
                                const size_t f = static_cast<size_t>(i2) * t.k + j;
                                if (!t.active[f]) continue;
                                if (t.n_spin == 0) sum += t.w[f];
                                else bp.h_dense_w[static_cast<size_t>(i2 * n_src + (t.idx[0][f] - ob.offset))] += t.w[f];
                            }
                            if (t.n_spin == 0) bp.h_dense_bias[i2] += sum;
                        }
                }
            }
        }
        CU_TRY(cudaStreamSynchronize(ctx->stream));  // host vectors above go out of scope
    }
    p->is_dense_source.assign(p->blocks.size(), 0);
    // A superblock is updated in place unless one of its blocks reads a position that the superblock writes
    // (several blocks updated "at the same time", sampling.rs:40-59, or a block with edges inside itself).
    p->staged.assign(p->sampling_order.size(), 0);
    for (size_t g = 0; g < p->sampling_order.size(); ++g) {
        const auto& members = p->sampling_order[g];
        for (int32_t m : members) p->blocks[m].order = static_cast<int32_t>(g);
        int64_t rows = 0;
        bool hit = false;
        for (int32_t m : members) rows += p->blocks[m].n;
        for (int32_t m : members) {
            for (const SlotTable& t : b->tables[m]) {
                for (size_t tl = 0; tl < t.idx.size() && !hit; ++tl)
                    for (int32_t o : members) {
                        const BlockProg& ob = p->blocks[o];
                        if (ob.sd != t.tail_sd[tl]) continue;
                        const int32_t lo = static_cast<int32_t>(ob.offset), hi = static_cast<int32_t>(ob.offset + ob.n);
                        const auto& ix = t.idx[tl];
                        for (size_t f = 0; f < ix.size(); ++f)
                            if (t.active[f] && ix[f] >= lo && ix[f] < hi) { hit = true; break; }
                        if (hit) break;
                    }
                if (hit) break;
            }
            if (hit) break;
        }
        if (hit) {
            p->staged[g] = 1;
            p->max_stage_rows = std::max(p->max_stage_rows, rows);
        }
    }
    *out = p.release();
    return THRML_OK;
}
// Handles may be destroyed in any order (a garbage collector does not promise one): no destroy function touches
// its parent handle; each waits for the whole device instead of for the parent's stream.
void thrml_program_destroy(thrml_program* p) {
    if (!p) return;
    cudaSetDevice(p->device);
    cudaDeviceSynchronize();
    delete p;
}
// The derived tables (thresholds, entry lists, split field tables) of a block whose slot weights changed.
static int32_t rebuild_derived(thrml_program* p, BlockProg& bp) {
    if (bp.base_kernel == 1)
        if (int32_t rc = rebuild_lut(p, bp)) return rc;
    if (bp.base_kernel == 4 || bp.base_kernel == 6)
        if (int32_t rc = rebuild_seq(p, bp)) return rc;
    if (bp.base_kernel == 6)
        if (int32_t rc = rebuild_lut(p, bp)) return rc;
    return THRML_OK;
}
int32_t thrml_program_update_weights(thrml_program* p, int32_t block, int32_t t, const float* w) {
    if (!p || !w) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (block < 0 || block >= p->n_free) return fail(THRML_ERR_INVALID_ARG, "block index out of range");
    BlockProg& bp = p->blocks[block];
    if (t < 0 || t >= bp.n_tabs) return fail(THRML_ERR_INVALID_ARG, "table index out of range");
    if (bp.dense_on) return fail(THRML_ERR_UNSUPPORTED, "weights of a block on the dense path are fixed; create a new program to change them");
    bp.dense_src = -1;  // the cached dense matrix no longer matches the tables
    CU_TRY(cudaSetDevice(p->ctx->device));
    CU_TRY(cudaMemcpyAsync(bp.w_bufs[t]->p, w, bp.w_len[t] * 4, cudaMemcpyHostToDevice, p->ctx->stream));
    if (int32_t rc = rebuild_derived(p, bp)) return rc;
    CU_TRY(cudaStreamSynchronize(p->ctx->stream));
    return THRML_OK;
}
// Slot s of a table copies row rows[s] of its source group (program.rs:216-235); the group's rows repeat the factor's
// `period` parameter rows once per head group (discrete_ebm.rs:391-453).
__global__ void k_regather(const int32_t* rows, const float* param, int64_t period, int32_t wdim, float scale, int64_t n_slots, float* w) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_slots * wdim) return;
    const int64_t s = i / wdim, d = i % wdim;
    w[i] = __fmul_rn(scale, param[(static_cast<int64_t>(rows[s]) % period) * wdim + d]);
}
int32_t thrml_program_update_group(thrml_program* p, int32_t group, const float* w, int64_t period, int32_t wdim, float scale) {
    if (!p || !w) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (period < 1 || wdim < 1) return fail(THRML_ERR_INVALID_ARG, "period and wdim must be positive");
    CU_TRY(cudaSetDevice(p->ctx->device));
    cudaStream_t st = p->ctx->stream;
    DevBuf d_param;
    bool found = false, uploaded = false;
    for (int32_t bi = 0; bi < p->n_free; ++bi) {
        BlockProg& bp = p->blocks[bi];
        bool touched = false;
        for (int32_t t = 0; t < bp.n_tabs; ++t) {
            if (bp.src_group[t] != group) continue;
            if (bp.tab_wdim[t] != wdim) return fail(THRML_ERR_INVALID_ARG, "wdim does not match the group's weights per row");
            if (bp.dense_on) return fail(THRML_ERR_UNSUPPORTED, "weights of a block on the dense path are fixed; create a new program to change them");
            if (!uploaded) {
                if (int32_t rc = upload(d_param, w, static_cast<size_t>(period) * wdim * 4, st)) return rc;
                uploaded = true;
            }
            const int64_t total = static_cast<int64_t>(bp.w_len[t]);
            k_regather<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(bp.rows_bufs[t]->as<int32_t>(), d_param.as<float>(), period, wdim, scale, total / wdim,
                                                                                 bp.w_bufs[t]->as<float>());
            CU_TRY(cudaGetLastError());
            found = touched = true;
        }
        if (touched) {
            bp.dense_src = -1;
            if (int32_t rc = rebuild_derived(p, bp)) return rc;
        }
    }
    CU_TRY(cudaStreamSynchronize(st));  // d_param is released on return
    if (!found) return fail(THRML_ERR_INVALID_ARG, "no free block has a table compiled from interaction group " + std::to_string(group));
    return THRML_OK;
}
int32_t thrml_program_enable_dense(thrml_program* p, int32_t allow_bf16_rounding, int32_t* n_blocks_out) {
    if (!p) return fail(THRML_ERR_INVALID_ARG, "null program");
    CU_TRY(cudaSetDevice(p->device));
    cudaStream_t st = p->ctx->stream;
    int32_t switched = 0;
    for (int32_t bi = 0; bi < p->n_free; ++bi) {
        BlockProg& bp = p->blocks[bi];
        if (bp.dense_src < 0 || bp.dense_on) continue;
        if (p->staged[bp.order]) continue;  // blocks updated through staging rows keep the gather kernel
        const int64_t n_src = p->blocks[bp.dense_src].n;
        bool exact = true;
        for (float w : bp.h_dense_w)
            if (bf16_to_f32(f32_to_bf16_rn(w)) != w) { exact = false; break; }
        if (!exact && !allow_bf16_rounding)
            return fail(THRML_ERR_INVALID_ARG, "the dense path stores couplings as bf16 and block " + std::to_string(bi) + " has couplings that are not bf16 values; pass allow_bf16_rounding = 1 to round them");
        bp.dense_pitch = (n_src + 63) / 64 * 64;
        std::vector<uint16_t> wb(static_cast<size_t>(bp.n * bp.dense_pitch), 0);
        for (int64_t i = 0; i < bp.n; ++i)
            for (int64_t j = 0; j < n_src; ++j) wb[static_cast<size_t>(i * bp.dense_pitch + j)] = f32_to_bf16_rn(bp.h_dense_w[static_cast<size_t>(i * n_src + j)]);
        if (int32_t rc = upload(bp.d_dense_w, wb.data(), wb.size() * 2, st)) return rc;
        if (int32_t rc = upload(bp.d_dense_bias, bp.h_dense_bias.data(), bp.h_dense_bias.size() * 4, st)) return rc;
        CU_TRY(cudaStreamSynchronize(st));
        bp.dense_bn = bp.n >= 2048 ? 256 : 128;  // wide output blocks take 128x256 tiles: fewer operand bytes per flop
        if (int32_t rc = make_operand_map(&bp.map_w, bp.d_dense_w.p, false, n_src, bp.n, bp.dense_pitch * 2, bp.dense_bn)) return rc;
        bp.dense_bn_pair = pair_tile_width(bp.n);
        if (int32_t rc = make_operand_map(&bp.map_w_pair, bp.d_dense_w.p, false, n_src, bp.n, bp.dense_pitch * 2, bp.dense_bn_pair / 2)) return rc;
        bp.dense_on = true;
        bp.kernel = 3;
        p->is_dense_source[bp.dense_src] = 1;
        p->any_dense = true;
        ++p->kernel_epoch;
        ++switched;
    }
    if (n_blocks_out) *n_blocks_out = switched;
    return THRML_OK;
}
int32_t thrml_program_block_kernel(const thrml_program* p, int32_t block, int32_t* kind_out) {
    if (!p || !kind_out || block < 0 || block >= p->n_free) return fail(THRML_ERR_INVALID_ARG, "block index out of range");
    *kind_out = p->blocks[block].kernel;
    return THRML_OK;
}

// ---------------------------------------------------------------------------------------------------------
// State.
// ---------------------------------------------------------------------------------------------------------
int32_t thrml_state_create(thrml_program* p, int64_t n_chains, int64_t chain_offset, thrml_state** out) {
    if (!p || !out) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (n_chains <= 0) return fail(THRML_ERR_INVALID_ARG, "n_chains must be positive");
    if (chain_offset < 0 || (chain_offset & 15)) return fail(THRML_ERR_INVALID_ARG, "chain_offset must be a non-negative multiple of 16");
    if (chain_offset + n_chains > (1LL << 32)) return fail(THRML_ERR_INVALID_ARG, "global chain ids must stay below 2^32");
    CU_TRY(cudaSetDevice(p->ctx->device));
    auto s = std::make_unique<thrml_state>();
    s->prog = p;
    s->device = p->device;
    s->n_chains = n_chains;
    s->chain_offset = chain_offset;
    s->ld = (n_chains + 15) / 16 * 16;
    for (int32_t c = 0; c < p->n_classes; ++c) {
        if (int32_t rc = s->cls[c].alloc(static_cast<size_t>(p->class_size[c]) * s->ld)) return rc;
        CU_TRY(cudaMemsetAsync(s->cls[c].p, 0, s->cls[c].bytes, p->ctx->stream));
    }
    if (p->max_stage_rows > 0)
        if (int32_t rc = s->stage.alloc(static_cast<size_t>(p->max_stage_rows) * s->ld)) return rc;
    const size_t nb_all = p->blocks.size();
    s->image.resize(nb_all);
    s->ones.resize(nb_all);
    s->image_fresh.assign(nb_all, 0);
    s->ones_fresh.assign(nb_all, 0);
    s->map_image.resize(nb_all);
    s->image_rows = (n_chains + 127) / 128 * 128;
    CU_TRY(cudaStreamSynchronize(p->ctx->stream));
    *out = s.release();
    return THRML_OK;
}
void thrml_state_destroy(thrml_state* s) {
    if (!s) return;
    cudaSetDevice(s->device);
    cudaDeviceSynchronize();
    delete s;
}

static int32_t check_block(const thrml_state* s, int32_t block) {
    if (!s) return fail(THRML_ERR_INVALID_ARG, "null state");
    if (block < 0 || block >= s->prog->n_free + s->prog->n_clamped) return fail(THRML_ERR_INVALID_ARG, "block index out of range");
    return THRML_OK;
}
int32_t thrml_state_upload_u8(thrml_state* s, int32_t block, const uint8_t* host) {
    if (int32_t rc = check_block(s, block)) return rc;
    if (!host) return fail(THRML_ERR_INVALID_ARG, "null host buffer");
    const BlockProg& bp = s->prog->blocks[block];
    cudaStream_t st = s->prog->ctx->stream;
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    const size_t bytes = static_cast<size_t>(bp.n) * s->n_chains;
    if (int32_t rc = need_scratch(s, bytes)) return rc;
    CU_TRY(cudaMemcpyAsync(s->scratch.p, host, bytes, cudaMemcpyHostToDevice, st));
    dim3 grid(static_cast<unsigned>((bp.n + 31) / 32), static_cast<unsigned>((s->ld + 31) / 32));
    k_transpose_in<<<grid, dim3(32, 8), 0, st>>>(s->scratch.as<uint8_t>(), s->rows(bp.sd) + bp.offset * s->ld, bp.n, s->n_chains, s->ld);
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaStreamSynchronize(st));
    s->touch(block);
    return THRML_OK;
}
// Several blocks in one call: every copy and layout kernel is queued on the context's stream and the host waits once at
// the end instead of once per block.  hosts[i] is block blocks[i]'s [chain][node] byte array.
int32_t thrml_state_upload_u8_many(thrml_state* s, const int32_t* blocks, int32_t n_blocks, const uint8_t* const* hosts) {
    if (!s || n_blocks < 0 || (n_blocks > 0 && (!blocks || !hosts))) return fail(THRML_ERR_INVALID_ARG, "null argument");
    size_t most = 0;
    for (int32_t i = 0; i < n_blocks; ++i) {
        if (int32_t rc = check_block(s, blocks[i])) return rc;
        if (!hosts[i]) return fail(THRML_ERR_INVALID_ARG, "null host buffer");
        most = std::max(most, static_cast<size_t>(s->prog->blocks[blocks[i]].n) * s->n_chains);
    }
    cudaStream_t st = s->prog->ctx->stream;
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    if (int32_t rc = need_scratch(s, most)) return rc;
    for (int32_t i = 0; i < n_blocks; ++i) {
        const BlockProg& bp = s->prog->blocks[blocks[i]];
        // the scratch is reused block after block: stream order keeps each copy behind the previous block's transpose
        CU_TRY(cudaMemcpyAsync(s->scratch.p, hosts[i], static_cast<size_t>(bp.n) * s->n_chains, cudaMemcpyHostToDevice, st));
        dim3 grid(static_cast<unsigned>((bp.n + 31) / 32), static_cast<unsigned>((s->ld + 31) / 32));
        k_transpose_in<<<grid, dim3(32, 8), 0, st>>>(s->scratch.as<uint8_t>(), s->rows(bp.sd) + bp.offset * s->ld, bp.n, s->n_chains, s->ld);
        CU_TRY(cudaGetLastError());
        s->touch(blocks[i]);
    }
    CU_TRY(cudaStreamSynchronize(st));
    return THRML_OK;
}
// Spin blocks as bits, the mirror of thrml_sample_states_packed: bits[i] is block blocks[i]'s [node][word] u32 array, word w
// holding chains 32w .. 32w+31 (bit c & 31).  One bit per spin crosses the host link, and the device layout is already
// chains-innermost, so the expansion is a streaming kernel with no transpose.
int32_t thrml_state_upload_packed(thrml_state* s, const int32_t* blocks, int32_t n_blocks, const uint32_t* const* bits) {
    if (!s || n_blocks < 0 || (n_blocks > 0 && (!blocks || !bits))) return fail(THRML_ERR_INVALID_ARG, "null argument");
    const int64_t words = (s->n_chains + 31) / 32;
    size_t total = 0;
    for (int32_t i = 0; i < n_blocks; ++i) {
        if (int32_t rc = check_block(s, blocks[i])) return rc;
        if (!bits[i]) return fail(THRML_ERR_INVALID_ARG, "null host buffer");
        if (s->prog->blocks[blocks[i]].is_cat) return fail(THRML_ERR_UNSUPPORTED, "bit-packed upload is for spin blocks");
        total += static_cast<size_t>(s->prog->blocks[blocks[i]].n) * words * 4;
    }
    cudaStream_t st = s->prog->ctx->stream;
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    if (int32_t rc = need_scratch(s, total)) return rc;  // all blocks side by side: the copies need not wait for the kernels
    size_t at = 0;
    for (int32_t i = 0; i < n_blocks; ++i) {
        const BlockProg& bp = s->prog->blocks[blocks[i]];
        const size_t bytes = static_cast<size_t>(bp.n) * words * 4;
        uint32_t* stage = reinterpret_cast<uint32_t*>(s->scratch.as<uint8_t>() + at);
        CU_TRY(cudaMemcpyAsync(stage, bits[i], bytes, cudaMemcpyHostToDevice, st));
        const int64_t threads = bp.n * (s->ld >> 4);
        k_unpack_rows<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, st>>>(stage, words, bp.n, s->ld, s->n_chains, s->rows(bp.sd) + bp.offset * s->ld);
        CU_TRY(cudaGetLastError());
        s->touch(blocks[i]);
        at += bytes;
    }
    CU_TRY(cudaStreamSynchronize(st));
    return THRML_OK;
}
// ---------------------------------------------------------------------------------------------------------
// Upload without any allocation.
//
// Some hosts must not allocate device memory once they are running: the GPU's memory was handed to another runtime's
// pool at start-up so a late cudaMalloc can fail, or the host sits in a latency-sensitive loop where cudaMalloc's
// device-wide synchronisation would stall its other streams.  thrml_state_upload_u8 may grow its staging buffer with
// cudaMalloc; this variant stages the [chain][node] bytes in a fixed array that is part of the library image instead.
//
// The array costs THRML_STATIC_SCRATCH_BYTES on every GPU that loads the library, until the process exits.  In host
// code its name is only a handle for the runtime, not a device address, so the address is looked up once per device
// with cudaGetSymbolAddress (with that device current) on the first call there; make that first call before starting
// any stream capture.  All calls share the array and it keeps whatever the last call left in it; the transpose reads
// only the bytes this call has just copied, so nothing needs clearing.  Two calls whose GPU work overlaps (different
// contexts or threads on the same device) would race on it: issue them one after the other.
// ---------------------------------------------------------------------------------------------------------
constexpr size_t THRML_STATIC_SCRATCH_BYTES = size_t(4) << 20;
constexpr int THRML_STATIC_MAX_DEVICES = 64;
static __device__ __align__(256) uint8_t g_static_scratch[THRML_STATIC_SCRATCH_BYTES];
static uint8_t* g_static_scratch_addr[THRML_STATIC_MAX_DEVICES] = {};

int32_t thrml_state_upload_u8_static(thrml_state* s, int32_t block, const uint8_t* host) {
    if (int32_t rc = check_block(s, block)) return rc;
    if (!host) return fail(THRML_ERR_INVALID_ARG, "null host buffer");
    const BlockProg& bp = s->prog->blocks[block];
    const size_t bytes = static_cast<size_t>(bp.n) * s->n_chains;
    if (bytes > THRML_STATIC_SCRATCH_BYTES)
        return fail(THRML_ERR_INVALID_ARG, "block of " + std::to_string(bytes) + " bytes (nodes x chains) exceeds the static scratch of " +
                                               std::to_string(THRML_STATIC_SCRATCH_BYTES) + " bytes; use thrml_state_upload_u8");
    const int dev = s->device;
    if (dev < 0 || dev >= THRML_STATIC_MAX_DEVICES) return fail(THRML_ERR_UNSUPPORTED, "device index beyond the static scratch table");
    CU_TRY(cudaSetDevice(dev));
    if (!g_static_scratch_addr[dev]) {
        uint8_t* addr = nullptr;
        CU_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_static_scratch));
        g_static_scratch_addr[dev] = addr;
    }
    uint8_t* scratch = g_static_scratch_addr[dev];
    cudaStream_t st = s->prog->ctx->stream;
    CU_TRY(cudaMemcpyAsync(scratch, host, bytes, cudaMemcpyHostToDevice, st));
    dim3 grid(static_cast<unsigned>((bp.n + 31) / 32), static_cast<unsigned>((s->ld + 31) / 32));
    k_transpose_in<<<grid, dim3(32, 8), 0, st>>>(scratch, s->rows(bp.sd) + bp.offset * s->ld, bp.n, s->n_chains, s->ld);
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaStreamSynchronize(st));
    s->touch(block);
    return THRML_OK;
}
int32_t thrml_state_download_u8(thrml_state* s, int32_t block, uint8_t* host) {
    if (int32_t rc = check_block(s, block)) return rc;
    if (!host) return fail(THRML_ERR_INVALID_ARG, "null host buffer");
    const BlockProg& bp = s->prog->blocks[block];
    cudaStream_t st = s->prog->ctx->stream;
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    const size_t bytes = static_cast<size_t>(bp.n) * s->n_chains;
    if (int32_t rc = need_scratch(s, bytes)) return rc;
    dim3 grid(static_cast<unsigned>((bp.n + 31) / 32), static_cast<unsigned>((s->n_chains + 31) / 32));
    k_transpose_out<<<grid, dim3(32, 8), 0, st>>>(s->rows(bp.sd) + bp.offset * s->ld, s->scratch.as<uint8_t>(), bp.n, s->n_chains, s->ld);
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaMemcpyAsync(host, s->scratch.p, bytes, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    return THRML_OK;
}
// A range of chains of one block, host layout [chain - chain_begin][node].
int32_t thrml_state_download_chains_u8(thrml_state* s, int32_t block, int64_t chain_begin, int64_t n_chains, uint8_t* host) {
    if (int32_t rc = check_block(s, block)) return rc;
    if (!host) return fail(THRML_ERR_INVALID_ARG, "null host buffer");
    if (chain_begin < 0 || n_chains < 1 || chain_begin + n_chains > s->n_chains) return fail(THRML_ERR_INVALID_ARG, "chain range out of the state");
    const BlockProg& bp = s->prog->blocks[block];
    cudaStream_t st = s->prog->ctx->stream;
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    const size_t bytes = static_cast<size_t>(bp.n) * n_chains;
    if (int32_t rc = need_scratch(s, bytes)) return rc;
    dim3 grid(static_cast<unsigned>((bp.n + 31) / 32), static_cast<unsigned>((n_chains + 31) / 32));
    k_transpose_out<<<grid, dim3(32, 8), 0, st>>>(s->rows(bp.sd) + bp.offset * s->ld + chain_begin, s->scratch.as<uint8_t>(), bp.n, n_chains, s->ld);
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaMemcpyAsync(host, s->scratch.p, bytes, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    return THRML_OK;
}
int32_t thrml_state_upload_f32(thrml_state* s, int32_t block, const float* host) {
    if (int32_t rc = check_block(s, block)) return rc;
    if (!host) return fail(THRML_ERR_INVALID_ARG, "null host buffer");
    const BlockProg& bp = s->prog->blocks[block];
    const size_t cnt = static_cast<size_t>(bp.n) * s->n_chains;
    std::vector<uint8_t> tmp(cnt);
    const float top = bp.is_cat ? static_cast<float>(bp.kind - 1) : 1.0f;
    for (size_t i = 0; i < cnt; ++i) {
        const float v = host[i];
        if (!(v >= 0.0f && v <= top) || v != static_cast<float>(static_cast<int>(v)))
            return fail(THRML_ERR_INVALID_ARG, bp.is_cat ? "categorical state must be an integer in [0, K)" : "spin state must be 0 or 1");
        tmp[i] = static_cast<uint8_t>(v);
    }
    return thrml_state_upload_u8(s, block, tmp.data());
}
int32_t thrml_state_download_f32(thrml_state* s, int32_t block, float* host) {
    if (int32_t rc = check_block(s, block)) return rc;
    if (!host) return fail(THRML_ERR_INVALID_ARG, "null host buffer");
    const BlockProg& bp = s->prog->blocks[block];
    const size_t cnt = static_cast<size_t>(bp.n) * s->n_chains;
    std::vector<uint8_t> tmp(cnt);
    if (int32_t rc = thrml_state_download_u8(s, block, tmp.data())) return rc;
    for (size_t i = 0; i < cnt; ++i) host[i] = static_cast<float>(tmp[i]);
    return THRML_OK;
}

int32_t thrml_hinton_init(thrml_state* s, const int32_t* blocks, int32_t n_blocks, const float* biases, float beta, uint64_t key, const float* inj_u) {
    if (!s || n_blocks < 0 || (n_blocks > 0 && (!blocks || !biases))) return fail(THRML_ERR_INVALID_ARG, "bad hinton_init arguments");
    cudaStream_t st = s->prog->ctx->stream;
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    std::vector<uint64_t> keys(static_cast<size_t>(n_blocks));
    rng_split(key, n_blocks, keys.data());  // ising.rs:618
    int64_t total = 0;
    for (int32_t i = 0; i < n_blocks; ++i) {
        if (int32_t rc = check_block(s, blocks[i])) return rc;
        if (s->prog->blocks[blocks[i]].is_cat) return fail(THRML_ERR_INVALID_ARG, "hinton_init applies to spin blocks");
        total += s->prog->blocks[blocks[i]].n;
    }
    const size_t bias_bytes = static_cast<size_t>(total) * 4, inj_bytes = inj_u ? static_cast<size_t>(total) * s->n_chains * 4 : 0;
    if (int32_t rc = need_scratch(s, bias_bytes + inj_bytes)) return rc;
    float* d_bias = s->scratch.as<float>();
    float* d_inj = inj_u ? d_bias + total : nullptr;
    CU_TRY(cudaMemcpyAsync(d_bias, biases, bias_bytes, cudaMemcpyHostToDevice, st));
    if (inj_u) CU_TRY(cudaMemcpyAsync(d_inj, inj_u, inj_bytes, cudaMemcpyHostToDevice, st));
    int64_t boff = 0;
    for (int32_t i = 0; i < n_blocks; ++i) {
        const BlockProg& bp = s->prog->blocks[blocks[i]];
        k_hinton<<<grid_nq(bp.n, s->ld), block_nq(s->ld), 0, st>>>(s->rows(bp.sd) + bp.offset * s->ld, s->ld, s->n_chains, static_cast<int32_t>(bp.n), d_bias + boff, beta,
                                                                 static_cast<uint32_t>(s->chain_offset >> 2), static_cast<uint32_t>(keys[i]),
                                                                 static_cast<uint32_t>(keys[i] >> 32), d_inj ? d_inj + boff * s->n_chains : nullptr);
        CU_TRY(cudaGetLastError());
        s->touch(blocks[i]);
        boff += bp.n;
    }
    CU_TRY(cudaStreamSynchronize(st));
    return THRML_OK;
}
int32_t thrml_state_randomize(thrml_state* s, uint64_t key) {
    if (!s) return fail(THRML_ERR_INVALID_ARG, "null state");
    cudaStream_t st = s->prog->ctx->stream;
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    const int32_t nf = s->prog->n_free;
    std::vector<uint64_t> keys(static_cast<size_t>(nf));
    rng_split(key, nf, keys.data());
    for (int32_t b = 0; b < nf; ++b) {
        const BlockProg& bp = s->prog->blocks[b];
        k_randomize<<<grid_nq(bp.n, s->ld), block_nq(s->ld), 0, st>>>(s->rows(bp.sd) + bp.offset * s->ld, s->ld, s->n_chains, static_cast<int32_t>(bp.n), bp.kind,
                                                                    static_cast<uint32_t>(s->chain_offset >> 2), static_cast<uint32_t>(keys[b]),
                                                                    static_cast<uint32_t>(keys[b] >> 32));
        CU_TRY(cudaGetLastError());
        s->touch(b);
    }
    CU_TRY(cudaStreamSynchronize(st));
    return THRML_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Sweeps.
// ---------------------------------------------------------------------------------------------------------
struct NoiseCursor {
    const float* u = nullptr;
    int64_t len = 0, pos = 0;
};

// ---- dense path plumbing -------------------------------------------------------------------------------
static int32_t ensure_err_flag(thrml_state* s) {
    if (s->d_err.p) return THRML_OK;
    if (int32_t rc = s->d_err.alloc(sizeof(int))) return rc;
    CU_TRY(cudaMemsetAsync(s->d_err.p, 0, sizeof(int), s->prog->ctx->stream));
    if (int32_t rc = s->d_dense_debug.alloc(2 * sizeof(uint32_t))) return rc;
    CU_TRY(cudaMemsetAsync(s->d_dense_debug.p, 0xff, 2 * sizeof(uint32_t), s->prog->ctx->stream));
    return THRML_OK;
}
// Reads the kernels' error flag after a synchronisation; a non-zero value means a bounded wait ran out.
static int32_t check_err_flag(thrml_state* s) {
    if (!s->d_err.p) return THRML_OK;
    int code = 0;
    CU_TRY(cudaMemcpy(&code, s->d_err.p, sizeof(int), cudaMemcpyDeviceToHost));
    if (code == 0) return THRML_OK;
    CU_TRY(cudaMemset(s->d_err.p, 0, sizeof(int)));
    return fail(THRML_ERR_TIMEOUT, "a tensor-core kernel gave up waiting on a pipeline barrier (role " + std::to_string(code) + ")");
}
// +-1 bf16 image [chain][node] of a block, rebuilt from the byte state when stale.
static int32_t ensure_image(thrml_state* s, int32_t block, bool need_fresh) {
    const BlockProg& bp = s->prog->blocks[block];
    const int64_t pitch = (bp.n + 63) / 64 * 64;
    if (!s->image[block]) {
        s->image[block].reset(new DevBuf());
        if (int32_t rc = s->image[block]->alloc(static_cast<size_t>(s->image_rows * pitch) * 2)) return rc;
        CU_TRY(cudaMemsetAsync(s->image[block]->p, 0, s->image[block]->bytes, s->prog->ctx->stream));
        if (int32_t rc = make_operand_map(&s->map_image[block], s->image[block]->p, false, bp.n, s->n_chains, pitch * 2, dense::BM)) return rc;
        s->image_fresh[block] = 0;
    }
    if (need_fresh && !s->image_fresh[block]) {
        // the same pass counts the ones per node when those are stale too (the correlation epilogue wants them)
        int32_t* ones = nullptr;
        if (!s->ones_fresh[block]) {
            if (!s->ones[block]) {
                s->ones[block].reset(new DevBuf());
                if (int32_t rc = s->ones[block]->alloc(static_cast<size_t>(bp.n) * 4)) return rc;
            }
            CU_TRY(cudaMemsetAsync(s->ones[block]->p, 0, static_cast<size_t>(bp.n) * 4, s->prog->ctx->stream));
            ones = s->ones[block]->as<int32_t>();
        }
        dim3 grid(static_cast<unsigned>(pitch / 32), static_cast<unsigned>((s->n_chains + 127) / 128));
        dense::k_make_image<<<grid, 256, 0, s->prog->ctx->stream>>>(s->rows(bp.sd) + bp.offset * s->ld, s->ld, s->n_chains, static_cast<int32_t>(bp.n),
                                                                    s->image[block]->as<__nv_bfloat16>(), pitch, ones);
        CU_TRY(cudaGetLastError());
        s->image_fresh[block] = 1;
        if (ones) s->ones_fresh[block] = 1;
    }
    return THRML_OK;
}
extern "C++" {
template <int EPI, int BN>
static int32_t launch_dense(thrml_state* s, const CUtensorMap& ma, const CUtensorMap& mb, dense::GemmArgs g) {
    constexpr size_t smem = dense::stages_for<BN>() * (dense::BM + BN) * dense::BK_BYTES + 1024;
    static bool configured[64] = {};  // the attribute is per device
    const int dev = s->device & 63;
    if (!configured[dev]) {
        CU_TRY(cudaFuncSetAttribute(dense::k_dense_gemm<EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured[dev] = true;
    }
    g.tiles_m = (g.m_total + dense::BM - 1) / dense::BM;
    g.tiles_n = (g.n_total + BN - 1) / BN;
    g.err = s->d_err.as<int>();
    const int ctas = std::min(s->prog->ctx->sm_count, g.tiles_m * g.tiles_n);
    dense::k_dense_gemm<EPI, BN><<<ctas, dense::THREADS, smem, s->prog->ctx->stream>>>(ma, mb, g);
    CU_TRY(cudaGetLastError());
    return THRML_OK;
}
template <int EPI, int BN>
static int32_t launch_dense_pair(thrml_state* s, const CUtensorMap& ma, const CUtensorMap& mb, dense::GemmArgs g) {
    constexpr size_t smem = dense::pair_stages_for<BN>() * (dense::BM + BN / 2) * dense::BK_BYTES + 1024;
    static bool configured[64] = {};  // the attribute is per device
    const int dev = s->device & 63;
    if (!configured[dev]) {
        CU_TRY(cudaFuncSetAttribute(dense::k_dense_gemm_pair<EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured[dev] = true;
    }
    g.tiles_m = (g.m_total + dense::PAIR_BM - 1) / dense::PAIR_BM;
    g.tiles_n = (g.n_total + BN - 1) / BN;
    g.err = s->d_err.as<int>();
    g.debug = s->d_dense_debug.as<uint32_t>();
    const int pairs = std::max(1, std::min(s->prog->ctx->sm_count / 2, g.tiles_m * g.tiles_n));
    dense::k_dense_gemm_pair<EPI, BN><<<2 * pairs, dense::THREADS, smem, s->prog->ctx->stream>>>(ma, mb, g);
    CU_TRY(cudaGetLastError());
    return THRML_OK;
}
}  // extern "C++"
// Tensor-core update of a dense bipartite block, in place; with `fields` the same GEMM writes the local fields
// (bias + accumulator, [chain][node] f32) instead of sampling.
extern "C++" {
template <int EPI>
static int32_t dense_launch_any(thrml_state* s, const BlockProg& bp, const dense::GemmArgs& g, const thrml_state* image_from = nullptr) {
    thrml_program* p = s->prog;
    const CUtensorMap& src = (image_from ? image_from : s)->map_image[bp.dense_src];  // the +-1 image of the neighbour block
    if (use_pair_tiles(p->dense_tiles, s->n_chains, p->blocks[bp.dense_src].n)) {
        if (bp.dense_bn_pair == 256) return launch_dense_pair<EPI, 256>(s, src, bp.map_w_pair, g);
        if (bp.dense_bn_pair == 208) return launch_dense_pair<EPI, 208>(s, src, bp.map_w_pair, g);
        return launch_dense_pair<EPI, 128>(s, src, bp.map_w_pair, g);
    }
    if (bp.dense_bn == 256) return launch_dense<EPI, 256>(s, src, bp.map_w, g);
    return launch_dense<EPI, 128>(s, src, bp.map_w, g);
}
}  // extern "C++"
static int32_t dense_fields(thrml_state* s, int32_t block, float* d_fields) {
    thrml_program* p = s->prog;
    const BlockProg& bp = p->blocks[block];
    if (int32_t rc = ensure_err_flag(s)) return rc;
    if (int32_t rc = ensure_image(s, bp.dense_src, true)) return rc;
    dense::GemmArgs g{};
    g.m_total = static_cast<int32_t>(s->n_chains);
    g.n_total = static_cast<int32_t>(bp.n);
    g.k_bytes = static_cast<int32_t>(p->blocks[bp.dense_src].n * 2);
    g.bias = bp.d_dense_bias.as<float>();
    g.fields_out = d_fields;
    return dense_launch_any<dense::EPI_FIELDS>(s, bp, g);
}
// `neighbours_from` (nullable): another state of the same program and chain count whose copy of the neighbour block is read
// instead of this state's.
static int32_t dense_update(thrml_state* s, int32_t block, uint32_t k0, uint32_t k1, thrml_state* neighbours_from = nullptr) {
    thrml_program* p = s->prog;
    const BlockProg& bp = p->blocks[block];
    if (int32_t rc = ensure_err_flag(s)) return rc;
    if (int32_t rc = ensure_image(neighbours_from ? neighbours_from : s, bp.dense_src, true)) return rc;
    const bool write_image = p->is_dense_source[block] != 0 && block != s->no_image_block;
    if (write_image)
        if (int32_t rc = ensure_image(s, block, false)) return rc;
    dense::GemmArgs g{};
    g.m_total = static_cast<int32_t>(s->n_chains);
    g.n_total = static_cast<int32_t>(bp.n);
    g.k_bytes = static_cast<int32_t>(p->blocks[bp.dense_src].n * 2);
    g.bias = bp.d_dense_bias.as<float>();
    g.state_out = s->rows(bp.sd) + bp.offset * s->ld;
    g.ld = s->ld;
    g.image_out = write_image ? s->image[block]->as<__nv_bfloat16>() : nullptr;
    g.image_pitch = (bp.n + 63) / 64 * 64;
    g.chain_word0 = static_cast<uint32_t>(s->chain_offset >> 2);
    g.rk = make_round_keys(static_cast<uint64_t>(k0) | (static_cast<uint64_t>(k1) << 32));
    if (!s->ones[block]) {
        s->ones[block].reset(new DevBuf());
        if (int32_t rc = s->ones[block]->alloc(static_cast<size_t>(bp.n) * 4)) return rc;
    }
    CU_TRY(cudaMemsetAsync(s->ones[block]->p, 0, static_cast<size_t>(bp.n) * 4, p->ctx->stream));
    g.ones_out = s->ones[block]->as<int32_t>();
    if (int32_t rc = dense_launch_any<dense::EPI_SAMPLE>(s, bp, g, neighbours_from)) return rc;
    s->image_fresh[block] = write_image ? 1 : 0;
    s->ones_fresh[block] = 1;
    return THRML_OK;
}

// One block update (program.rs:324-393 + the sampler), asynchronous on the context's stream.  mode 0 sample, 2 fields.
static int32_t launch_block(thrml_state* s, int32_t block, uint64_t key, NoiseCursor* inj, uint8_t* dst, float* fields, thrml_moments* acc = nullptr) {
    thrml_program* p = s->prog;
    const BlockProg& bp = p->blocks[block];
    cudaStream_t st = p->ctx->stream;
    const uint32_t k0 = static_cast<uint32_t>(key), k1 = static_cast<uint32_t>(key >> 32);
    const uint32_t word0 = static_cast<uint32_t>(s->chain_offset >> 2);
    const bool to_state = dst == s->rows(bp.sd) + bp.offset * s->ld;
    if (!fields) ++s->block_launches;
    if (bp.kernel == 3 && !inj && !fields && to_state) {
        if (int32_t rc = dense_update(s, block, k0, k1)) return rc;
        return THRML_OK;
    }
    if (!fields) s->touch(block);
    if (bp.base_kernel == 1 && !inj && !fields) {
        LutArgs a{bp.d_nbr.as<int32_t>(), bp.d_lut.as<uint32_t>(), s->rows(p->sd_spin), dst, s->ld, static_cast<int32_t>(bp.n), static_cast<int32_t>(s->ld / 16), word0,
                  make_round_keys(key), s->n_chains, nullptr, nullptr, nullptr};
        const bool few_chains = a.n_chunks <= FEW_CHAIN_CHUNKS;  // a thread per (node, 16 chains) instead of a warp per node
        const int64_t ctas = few_chains ? std::min<int64_t>((bp.n * a.n_chunks + 255) / 256, static_cast<int64_t>(p->ctx->sm_count) * 16)
                                        : std::min<int64_t>((bp.n + 7) / 8, static_cast<int64_t>(p->ctx->sm_count) * 8);
        if (acc && acc->fused[block]) {
            a.m1_row = acc->fused[block]->m1.as<int32_t>();
            a.m2_row = acc->fused[block]->m2.as<int32_t>();
            a.sums = acc->d_sums.as<long long>();
            if (few_chains) k_spin_lut_thread<true><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
            else k_spin_lut<true><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
        } else if (few_chains) {
            k_spin_lut_thread<false><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
        } else {
            k_spin_lut<false><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
        }
        CU_TRY(cudaGetLastError());
        return THRML_OK;
    }
    // With few chains the warp-per-node kernels idle most lanes (16 chains per lane); the node x quad gather kernel, which
    // then packs several nodes into a warp, is the faster one unless the observer has to ride along.
    const bool narrow = s->ld / 16 <= NARROW_CHUNKS && !(acc && acc->fused[block]);
    if (bp.base_kernel == 6 && !inj && !fields && !narrow) {
        HybridArgs a{};
        a.lut = LutArgs{bp.d_nbr.as<int32_t>(), bp.d_lut.as<uint32_t>(), s->rows(p->sd_spin), dst, s->ld, static_cast<int32_t>(bp.n), static_cast<int32_t>(s->ld / 16), word0,
                        make_round_keys(key), s->n_chains, nullptr, nullptr, nullptr};
        a.seq = SeqArgs{bp.d_seq_nbr.as<int32_t>(), bp.d_seq_w.as<float>(), bp.d_seq_first.as<uint32_t>(), bp.d_seq_cnt.as<int32_t>(), bp.d_seq_overflow.as<int32_t>(),
                        bp.d_seq_n_rows.as<int32_t>(), s->rows(p->sd_spin), dst, s->ld,
                        static_cast<int32_t>(bp.n), static_cast<int32_t>(s->ld / 16), word0, a.lut.rk, s->n_chains, nullptr, nullptr, nullptr, nullptr, nullptr};
        a.lut_row = bp.d_lut_row.as<int32_t>();
        a.seq.order = bp.d_seq_order.as<int32_t>();
        a.seq.counter = bp.d_seq_counter.as<int32_t>();
        if (bp.n_split > 0 && a.seq.n_chunks >= SPLIT_MIN_CHUNKS) {
            a.seq.split_row = bp.d_split_row.as<int32_t>();
            a.seq.split_tab = bp.d_split_tab.as<float>();
            a.seq.split_margin = bp.d_split_margin.as<float>();
        }
        CU_TRY(cudaMemsetAsync(a.seq.counter, 0, 4, st));
        const int64_t ctas = std::min<int64_t>((bp.n + 7) / 8, static_cast<int64_t>(p->ctx->sm_count) * 8);
        if (acc && acc->fused[block]) {
            a.lut.m1_row = a.seq.m1_row = acc->fused[block]->m1.as<int32_t>();
            a.lut.m2_row = a.seq.m2_row = acc->fused[block]->m2.as<int32_t>();
            a.lut.sums = a.seq.sums = acc->d_sums.as<long long>();
            if (bp.split_wide) k_spin_hybrid<true, true><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
            else k_spin_hybrid<true, false><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
        } else if (bp.split_wide) {
            k_spin_hybrid<false, true><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
        } else {
            k_spin_hybrid<false, false><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
        }
        CU_TRY(cudaGetLastError());
        return THRML_OK;
    }
    if (bp.base_kernel == 4 && !inj && !fields && !narrow) {
        SeqArgs a{bp.d_seq_nbr.as<int32_t>(), bp.d_seq_w.as<float>(), bp.d_seq_first.as<uint32_t>(), bp.d_seq_cnt.as<int32_t>(), bp.d_seq_overflow.as<int32_t>(),
                  bp.d_seq_n_rows.as<int32_t>(), s->rows(p->sd_spin), dst, s->ld,
                  static_cast<int32_t>(bp.n), static_cast<int32_t>(s->ld / 16), word0, make_round_keys(key), s->n_chains, nullptr, nullptr, nullptr,
                  bp.d_seq_order.as<int32_t>(), bp.d_seq_counter.as<int32_t>(), nullptr, nullptr, nullptr};
        if (bp.n_split > 0 && a.n_chunks >= SPLIT_MIN_CHUNKS) {
            a.split_row = bp.d_split_row.as<int32_t>();
            a.split_tab = bp.d_split_tab.as<float>();
            a.split_margin = bp.d_split_margin.as<float>();
        }
        CU_TRY(cudaMemsetAsync(a.counter, 0, 4, st));
        const int64_t ctas = std::min<int64_t>((bp.n + 7) / 8, static_cast<int64_t>(p->ctx->sm_count) * 8);
        if (acc && acc->fused[block]) {
            a.m1_row = acc->fused[block]->m1.as<int32_t>();
            a.m2_row = acc->fused[block]->m2.as<int32_t>();
            a.sums = acc->d_sums.as<long long>();
            if (bp.split_wide) k_spin_seq<true, true><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
            else k_spin_seq<true, false><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
        } else if (bp.split_wide) {
            k_spin_seq<false, true><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
        } else {
            k_spin_seq<false, false><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
        }
        CU_TRY(cudaGetLastError());
        return THRML_OK;
    }
    if (bp.base_kernel == 7 && !inj && !fields && !narrow && !p->gather_only) {
        WideArgs a{bp.d_tabs.as<DevTable>(), bp.d_wide_ent.as<int32_t>(), bp.d_wide_first.as<uint32_t>(), bp.d_wide_cnt.as<int32_t>(),
                   p->sd_spin >= 0 ? s->rows(p->sd_spin) : nullptr, p->sd_cat >= 0 ? s->rows(p->sd_cat) : nullptr, dst, s->ld,
                   static_cast<int32_t>(bp.n), static_cast<int32_t>(s->ld / 16), word0, s->n_chains, make_round_keys(key)};
        const int64_t ctas = std::min<int64_t>((bp.n + 7) / 8, static_cast<int64_t>(p->ctx->sm_count) * 6);
        if (bp.wide_has_cat) k_spin_wide<true><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
        else k_spin_wide<false><<<static_cast<unsigned>(ctas), 256, 0, st>>>(a);
        CU_TRY(cudaGetLastError());
        return THRML_OK;
    }
    UpdateArgs a{};
    a.tabs = bp.d_tabs.as<DevTable>();
    a.n_tabs = bp.n_tabs;
    a.n = static_cast<int32_t>(bp.n);
    a.K = bp.kind;
    a.ld = s->ld;
    a.n_chains = s->n_chains;
    a.chain_word0 = word0;
    a.spin = p->sd_spin >= 0 ? s->rows(p->sd_spin) : nullptr;
    a.cat = p->sd_cat >= 0 ? s->rows(p->sd_cat) : nullptr;
    a.dst = dst;
    a.k0 = k0;
    a.k1 = k1;
    a.fields = fields;
    if (inj) {
        const int64_t need = bp.n * s->n_chains * (bp.is_cat ? bp.kind : 1);
        if (inj->pos + need > inj->len) return fail(THRML_ERR_INVALID_ARG, "injected noise is shorter than the updates it must feed");
        if (int32_t rc = need_scratch(s, static_cast<size_t>(need) * 4)) return rc;
        CU_TRY(cudaMemcpyAsync(s->scratch.p, inj->u + inj->pos, static_cast<size_t>(need) * 4, cudaMemcpyHostToDevice, st));
        inj->pos += need;
        a.inj = s->scratch.as<float>();
    }
    const dim3 grid = grid_nq(bp.n, s->ld), blk = block_nq(s->ld);
    if (bp.is_cat) {
        if (fields) k_cat_generic<2><<<grid, blk, 0, st>>>(a);
        else if (inj) k_cat_generic<1><<<grid, blk, 0, st>>>(a);
        else if (bp.kernel == 5 && !p->gather_only && bp.cat_warp && s->ld >= 128) {
            CatWarpArgs w{a, bp.d_wide_ent.as<int32_t>(), bp.d_wide_first.as<uint32_t>(), bp.d_wide_cnt.as<int32_t>(), static_cast<int32_t>(s->ld / 4), make_round_keys(key)};
            const int K = bp.kind, KP = (K + 3) & ~3;
            const size_t smem = static_cast<size_t>(8) * CAT_SLOTS * K * KP * 4;
            const unsigned ctas = static_cast<unsigned>(std::min<int64_t>((bp.n + 7) / 8, static_cast<int64_t>(p->ctx->sm_count) * 8));
            auto go = [&](auto kernel) -> int32_t {
                if (smem > 48 * 1024) CU_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
                kernel<<<ctas, 256, smem, st>>>(w);
                return THRML_OK;
            };
            int32_t rc;
            if (K <= 4) rc = go(k_cat_warp<4>);
            else if (K <= 8) rc = go(k_cat_warp<8>);
            else if (K <= 10) rc = go(k_cat_warp<10>);
            else if (K <= 12) rc = go(k_cat_warp<12>);
            else rc = go(k_cat_warp<16>);
            if (rc) return rc;
        }
        else if (bp.kernel == 8 && !p->gather_only && s->ld >= 128) {
            CatManyArgs w{CatWarpArgs{a, bp.d_wide_ent.as<int32_t>(), bp.d_wide_first.as<uint32_t>(), bp.d_wide_cnt.as<int32_t>(), static_cast<int32_t>(s->ld / 4), make_round_keys(key)},
                          bp.cat_most};
            // staged weights: `cat_most` rows of K x KP floats per warp; eight warps per CTA while two CTAs fit an SM, four
            // while one does, otherwise the weights are read through L1
            const int K = bp.kind, KP = (K + 3) & ~3;
            const size_t per_warp = static_cast<size_t>(bp.cat_most) * K * KP * 4;
            const int warps = per_warp * 8 <= 72 * 1024 ? 8 : (per_warp * 4 <= 160 * 1024 ? 4 : 0);
            const size_t smem = warps ? per_warp * warps : 0;
            const int wpc = warps ? warps : 8;
            const unsigned ctas = static_cast<unsigned>(std::min<int64_t>((bp.n + wpc - 1) / wpc, static_cast<int64_t>(p->ctx->sm_count) * 8));
            auto go = [&](auto kernel) -> int32_t {
                // the kernel's static arrays take 35 KiB: the opt-in is needed well below 48 KiB of dynamic memory
                if (smem > 8 * 1024) CU_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
                kernel<<<ctas, 32 * wpc, smem, st>>>(w);
                return THRML_OK;
            };
            int32_t rc;
            if (warps) {
                if (K <= 4) rc = go(k_cat_many<4, true>);
                else if (K <= 8) rc = go(k_cat_many<8, true>);
                else if (K <= 12) rc = go(k_cat_many<12, true>);
                else rc = go(k_cat_many<16, true>);
            } else {
                if (K <= 4) rc = go(k_cat_many<4, false>);
                else if (K <= 8) rc = go(k_cat_many<8, false>);
                else if (K <= 12) rc = go(k_cat_many<12, false>);
                else rc = go(k_cat_many<16, false>);
            }
            if (rc) return rc;
        }
        else if (bp.kernel == 5 && !p->gather_only) {
            // weight rows staged in shared memory when CAT_SLOTS x K x K floats per node of the CTA fit in 48 KiB
            const size_t smem = static_cast<size_t>(blk.y) * CAT_SLOTS * bp.kind * bp.kind * 4;
            if (smem <= 48 * 1024 && 32 % blk.x == 0) k_cat_fast<true><<<grid, blk, smem, st>>>(a);
            else k_cat_fast<false><<<grid, blk, 0, st>>>(a);
        }
        else k_cat_generic<0><<<grid, blk, 0, st>>>(a);
    } else {
        if (fields) k_spin_generic<2><<<grid, blk, 0, st>>>(a);
        else if (inj) k_spin_generic<1><<<grid, blk, 0, st>>>(a);
        else k_spin_generic<0><<<grid, blk, 0, st>>>(a);
    }
    CU_TRY(cudaGetLastError());
    if (inj) CU_TRY(cudaStreamSynchronize(st));  // the scratch slice is reused by the next block
    return THRML_OK;
}

static int32_t observe_async(thrml_moments* m, thrml_state* s);

// sample_blocks (sampling.rs:28-63), asynchronous.  With `acc` the sweep is followed by an observation of `acc`:
// the threshold-table kernels accumulate their rows while they update, one k_moments launch covers the other rows.
// Bit-packed route (THRML_OPT_STATE_FORMAT = 1): every free block on the threshold-table kernel, nothing staged, rows wide
// enough to fill a warp with words (1024 chains), and an observer (if any) whose rows the update kernels own entirely.
static bool packed_route(const thrml_state* s, const thrml_moments* acc) {
    const thrml_program* p = s->prog;
    if (p->state_format != 1 || p->sd_spin < 0 || p->n_free < 1 || s->ld < 1024) return false;
    for (size_t g = 0; g < p->sampling_order.size(); ++g) {
        if (p->staged[g]) return false;
        for (int32_t m : p->sampling_order[g])
            if (p->blocks[m].kernel != 1 || p->blocks[m].base_kernel != 1) return false;
    }
    if (acc && !(acc->mode == 0 && acc->any_fused && acc->n_left == 0 && acc->kernel_epoch == p->kernel_epoch && acc->prog == p)) return false;
    return true;
}
static int32_t sweep_packed(thrml_state* s, uint64_t key, thrml_moments* acc) {
    thrml_program* p = s->prog;
    std::vector<uint64_t> keys(static_cast<size_t>(p->n_free));
    rng_split(key, p->n_free, keys.data());
    cudaStream_t st = p->ctx->stream;
    uint32_t* rows = nullptr;
    if (int32_t rc = s->packed_rows(&rows)) return rc;
    for (const auto& members : p->sampling_order)
        for (int32_t m : members) {
            const BlockProg& bp = p->blocks[m];
            const bool f = acc && acc->fused[m];
            PackedArgs a{bp.d_nbr.as<int32_t>(), bp.d_lut.as<uint32_t>(), rows, rows + bp.offset * s->pw, s->pw, static_cast<int32_t>(bp.n),
                         static_cast<int32_t>((s->n_chains + 31) / 32), static_cast<uint32_t>(s->chain_offset >> 2), s->n_chains, make_round_keys(keys[m]),
                         f ? acc->fused[m]->m1.as<int32_t>() : nullptr, f ? acc->fused[m]->m2.as<int32_t>() : nullptr, f ? acc->d_sums.as<long long>() : nullptr};
            const unsigned ctas = static_cast<unsigned>(std::min<int64_t>((bp.n + 7) / 8, static_cast<int64_t>(p->ctx->sm_count) * 8));
            if (f) k_packed_lut<true><<<ctas, 256, 0, st>>>(a);
            else k_packed_lut<false><<<ctas, 256, 0, st>>>(a);
            CU_TRY(cudaGetLastError());
            s->touch(m);
            ++s->block_launches;
        }
    if (acc) acc->n_obs += s->n_chains;
    return THRML_OK;
}

static int32_t sweep(thrml_state* s, uint64_t key, NoiseCursor* inj, thrml_moments* acc = nullptr) {
    if (!inj && packed_route(s, acc)) return sweep_packed(s, key, acc);
    const bool fuse = acc && acc->mode == 0 && acc->any_fused && !inj && acc->kernel_epoch == s->prog->kernel_epoch;
    thrml_program* p = s->prog;
    std::vector<uint64_t> keys(static_cast<size_t>(p->n_free));
    rng_split(key, p->n_free, keys.data());
    cudaStream_t st = p->ctx->stream;
    for (size_t g = 0; g < p->sampling_order.size(); ++g) {
        const auto& members = p->sampling_order[g];
        if (!p->staged[g]) {
            for (int32_t m : members) {
                const BlockProg& bp = p->blocks[m];
                if (int32_t rc = launch_block(s, m, keys[m], inj, s->rows(bp.sd) + bp.offset * s->ld, nullptr, fuse ? acc : nullptr)) return rc;
            }
            continue;
        }
        int64_t row = 0;
        for (int32_t m : members) {
            if (int32_t rc = launch_block(s, m, keys[m], inj, s->stage.as<uint8_t>() + row * s->ld, nullptr, fuse ? acc : nullptr)) return rc;
            row += p->blocks[m].n;
        }
        row = 0;
        for (int32_t m : members) {  // all members written back together (sampling.rs:57-59)
            const BlockProg& bp = p->blocks[m];
            CU_TRY(cudaMemcpyAsync(s->rows(bp.sd) + bp.offset * s->ld, s->stage.as<uint8_t>() + row * s->ld, static_cast<size_t>(bp.n) * s->ld, cudaMemcpyDeviceToDevice, st));
            s->touch(m);
            row += bp.n;
        }
    }
    if (!acc) return THRML_OK;
    if (!fuse) return observe_async(acc, s);
    if (acc->n_left > 0) {
        const unsigned grid = static_cast<unsigned>((acc->n_left + 7) / 8);
        if (acc->left_all_spin)
            k_moments_spin<<<grid, dim3(32, 8), 0, st>>>(acc->d_left_ptr.as<int64_t>(), acc->d_left_pos.as<int32_t>(), acc->n_left, s->rows(p->sd_spin), s->ld, s->n_chains,
                                                         acc->d_sums.as<unsigned long long>(), acc->d_left_rows.as<int64_t>());
        else
            k_moments<<<grid, dim3(32, 8), 0, st>>>(acc->d_left_ptr.as<int64_t>(), acc->d_left_sd.as<int32_t>(), acc->d_left_pos.as<int32_t>(), acc->n_left, s->rows(0),
                                                    s->rows(1), s->ld, s->n_chains, acc->spin_transform, acc->d_sums.as<unsigned long long>(),
                                                    acc->d_left_rows.as<int64_t>());
        CU_TRY(cudaGetLastError());
    }
    acc->n_obs += s->n_chains;
    return THRML_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Persistent sweeps for small programs.
//
// When every free block runs the threshold-table kernel, nothing is staged and one sweep touches little enough
// state to live in L2, a block update takes a microsecond or two and a schedule of thousands of sweeps is bound
// by its launches.  run() then queues its sweeps instead of launching them, and the queue is flushed as ONE
// cooperative launch of k_spin_lut_persistent per PERSIST_MAX_STEPS block updates.  Results are the same bits:
// the same per-block keys, the same update function, a grid-wide barrier where a kernel boundary used to be.
constexpr int64_t PERSIST_MAX_SWEEP_BYTES = int64_t(8) << 20;  // nodes x chains updated by one sweep
constexpr size_t PERSIST_MAX_STEPS = 4096;
constexpr size_t SLICE_MAX_STEPS = 16384;     // block updates per launch of the chain-sliced kernel
constexpr size_t SLICE_MAX_SMEM = 200 * 1024;  // state words + observer partial sums of one chain slice

static int persistent_grid(thrml_state* s) {
    thrml_program* p = s->prog;
    if (s->persist_epoch == p->kernel_epoch) return s->persist_grid;
    s->persist_epoch = p->kernel_epoch;
    s->persist_grid = 0;
    int64_t bytes = 0, max_n = 0;
    for (size_t g = 0; g < p->sampling_order.size(); ++g) {
        if (p->staged[g]) return 0;
        for (int32_t m : p->sampling_order[g]) {
            const BlockProg& bp = p->blocks[m];
            if (bp.kernel != 1 || bp.base_kernel != 1) return 0;
            bytes += bp.n * s->ld;
            max_n = std::max(max_n, bp.n);
        }
    }
    if (p->n_free < 1 || bytes > PERSIST_MAX_SWEEP_BYTES) return 0;
    s->sliced = static_cast<size_t>(p->class_size[p->sd_spin]) * 4 <= SLICE_MAX_SMEM && p->n_free <= SLICE_MAX_BLOCKS;
    if (s->sliced) return s->persist_grid = 1;
    int coop = 0, per_sm = 0;
    if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, p->ctx->device) != cudaSuccess || !coop) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_spin_lut_persistent, 256, 0) != cudaSuccess || per_sm < 1) return 0;
    const int64_t resident = static_cast<int64_t>(per_sm) * p->ctx->sm_count;
    s->persist_grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(resident, (max_n + 7) / 8)));
    return s->persist_grid;
}
static bool observer_rides_along(const thrml_moments* acc, const thrml_state* s) {
    if (!(acc->mode == 0 && acc->any_fused && acc->n_left == 0 && acc->kernel_epoch == s->prog->kernel_epoch && acc->prog == s->prog)) return false;
    if (s->sliced && static_cast<size_t>(s->prog->class_size[s->prog->sd_spin] + acc->total_rows) * 4 > SLICE_MAX_SMEM) return false;
    for (const auto& sw : s->pending)  // one observer per queue
        if (sw.second && sw.second != acc) return false;
    return true;
}
static int32_t flush_sliced(thrml_state* s) {
    thrml_program* p = s->prog;
    cudaStream_t st = p->ctx->stream;
    thrml_moments* acc = nullptr;
    for (const auto& sw : s->pending)
        if (sw.second) acc = sw.second;
    std::vector<SliceBlock> blocks(static_cast<size_t>(p->n_free));
    const int64_t n_spin = p->class_size[p->sd_spin], n_rows = acc ? acc->total_rows : 0;
    int64_t max_n = 0, words = (n_spin + n_rows + 3) / 4 * 4;
    const int64_t base_words = words;
    for (int32_t m = 0; m < p->n_free; ++m) {
        const BlockProg& bp = p->blocks[m];
        const bool f = acc && acc->fused[m];
        blocks[m] = SliceBlock{bp.d_nbr.as<int32_t>(), bp.d_lut.as<uint32_t>(), f ? acc->fused[m]->m1.as<int32_t>() : nullptr, f ? acc->fused[m]->m2.as<int32_t>() : nullptr,
                               static_cast<int32_t>(bp.n), static_cast<int32_t>(bp.offset), bp.max_deg, static_cast<int32_t>(words)};
        words += slice_block_words(bp.n, bp.max_deg, f);
        max_n = std::max(max_n, bp.n);
    }
    const bool resident = static_cast<size_t>(words) * 4 <= SLICE_MAX_SMEM;
    std::vector<SliceStep> steps;
    std::vector<uint64_t> keys(static_cast<size_t>(p->n_free));
    steps.reserve(s->pending.size() * static_cast<size_t>(p->n_free));
    for (const auto& sw : s->pending) {
        rng_split(sw.first, p->n_free, keys.data());
        for (const auto& members : p->sampling_order)
            for (int32_t m : members) steps.push_back(SliceStep{m, sw.second && blocks[m].m1_row ? 1 : 0, make_round_keys(keys[m])});
        if (sw.second) sw.second->n_obs += s->n_chains;
    }
    s->pending.clear();
    for (int32_t m = 0; m < p->n_free; ++m) s->touch(m);
    if (!s->d_slice_blocks.holds(blocks.size() * sizeof(SliceBlock)))
        if (int32_t rc = s->d_slice_blocks.alloc(blocks.size() * sizeof(SliceBlock))) return rc;
    if (!s->d_plan.holds(steps.size() * sizeof(SliceStep)))
        if (int32_t rc = s->d_plan.alloc(std::max(steps.size() * sizeof(SliceStep), PERSIST_MAX_STEPS * sizeof(LutArgs)))) return rc;
    // pageable sources: the copies have been staged by the time the calls return
    CU_TRY(cudaMemcpyAsync(s->d_slice_blocks.p, blocks.data(), blocks.size() * sizeof(SliceBlock), cudaMemcpyHostToDevice, st));
    CU_TRY(cudaMemcpyAsync(s->d_plan.p, steps.data(), steps.size() * sizeof(SliceStep), cudaMemcpyHostToDevice, st));
    SliceArgs a{s->d_slice_blocks.as<SliceBlock>(), s->d_plan.as<SliceStep>(), p->n_free, static_cast<int32_t>(steps.size()), static_cast<int32_t>(n_spin),
                static_cast<int32_t>(n_rows), resident ? 1 : 0, static_cast<uint32_t>(s->chain_offset >> 2), s->rows(p->sd_spin), s->ld, s->n_chains,
                acc ? acc->d_sums.as<unsigned long long>() : nullptr};
    const size_t smem = static_cast<size_t>(resident ? words : base_words) * 4;
    static bool configured[64] = {};  // the attribute is per device
    if (!configured[s->device & 63]) {
        CU_TRY(cudaFuncSetAttribute(k_spin_lut_sliced<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SLICE_MAX_SMEM)));
        CU_TRY(cudaFuncSetAttribute(k_spin_lut_sliced<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(SLICE_MAX_SMEM)));
        configured[s->device & 63] = true;
    }
    const int threads = static_cast<int>(std::min<int64_t>(512, std::max<int64_t>(64, (max_n + 31) / 32 * 32)));
    const unsigned grid = static_cast<unsigned>((s->n_chains + 3) / 4);
    if (resident) k_spin_lut_sliced<true><<<grid, threads, smem, st>>>(a);
    else k_spin_lut_sliced<false><<<grid, threads, smem, st>>>(a);
    CU_TRY(cudaGetLastError());
    ++s->persistent_launches;
    return THRML_OK;
}
static int32_t flush_pending(thrml_state* s) {
    if (s->pending.empty()) return THRML_OK;
    if (s->sliced) return flush_sliced(s);
    thrml_program* p = s->prog;
    cudaStream_t st = p->ctx->stream;
    const uint32_t word0 = static_cast<uint32_t>(s->chain_offset >> 2);
    std::vector<LutArgs> steps;
    std::vector<uint8_t> accf;
    std::vector<uint64_t> keys(static_cast<size_t>(p->n_free));
    steps.reserve(s->pending.size() * static_cast<size_t>(p->n_free));
    for (const auto& sw : s->pending) {
        rng_split(sw.first, p->n_free, keys.data());
        thrml_moments* acc = sw.second;
        for (const auto& members : p->sampling_order)
            for (int32_t m : members) {
                const BlockProg& bp = p->blocks[m];
                LutArgs a{bp.d_nbr.as<int32_t>(), bp.d_lut.as<uint32_t>(), s->rows(p->sd_spin), s->rows(bp.sd) + bp.offset * s->ld, s->ld, static_cast<int32_t>(bp.n),
                          static_cast<int32_t>(s->ld / 16), word0, make_round_keys(keys[m]), s->n_chains, nullptr, nullptr, nullptr};
                uint8_t f = 0;
                if (acc && acc->fused[m]) {
                    a.m1_row = acc->fused[m]->m1.as<int32_t>();
                    a.m2_row = acc->fused[m]->m2.as<int32_t>();
                    a.sums = acc->d_sums.as<long long>();
                    f = 1;
                }
                steps.push_back(a);
                accf.push_back(f);
            }
        if (acc) acc->n_obs += s->n_chains;
    }
    s->pending.clear();
    for (int32_t m = 0; m < p->n_free; ++m) s->touch(m);
    const int grid = s->persist_grid;
    for (size_t at = 0; at < steps.size(); at += PERSIST_MAX_STEPS) {
        const size_t cnt = std::min(PERSIST_MAX_STEPS, steps.size() - at);
        if (!s->d_plan.holds(cnt * sizeof(LutArgs)))
            if (int32_t rc = s->d_plan.alloc(PERSIST_MAX_STEPS * sizeof(LutArgs))) return rc;
        if (!s->d_plan_acc.holds(cnt))
            if (int32_t rc = s->d_plan_acc.alloc(PERSIST_MAX_STEPS)) return rc;
        // pageable sources: both copies have been staged by the time the calls return, so `steps` may be reused
        CU_TRY(cudaMemcpyAsync(s->d_plan.p, steps.data() + at, cnt * sizeof(LutArgs), cudaMemcpyHostToDevice, st));
        CU_TRY(cudaMemcpyAsync(s->d_plan_acc.p, accf.data() + at, cnt, cudaMemcpyHostToDevice, st));
        const LutArgs* d_steps = s->d_plan.as<LutArgs>();
        const uint8_t* d_acc = s->d_plan_acc.as<uint8_t>();
        int32_t n_steps = static_cast<int32_t>(cnt);
        void* args[] = {&d_steps, &d_acc, &n_steps};
        CU_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(k_spin_lut_persistent), dim3(static_cast<unsigned>(grid)), dim3(256), args, 0, st));
        ++s->persistent_launches;
    }
    return THRML_OK;
}

// run_blocks (sampling.rs:81-106), asynchronous; `acc` (nullable) is observed after the last sweep.
static int32_t run(thrml_state* s, uint64_t key, int64_t n_iters, NoiseCursor* inj, thrml_moments* acc = nullptr) {
    if (n_iters <= 0) return acc ? observe_async(acc, s) : THRML_OK;
    std::vector<uint64_t> keys(static_cast<size_t>(n_iters));
    rng_split(key, n_iters, keys.data());
    const bool queue = !inj && !packed_route(s, nullptr) && persistent_grid(s) > 0;  // an explicit bit-packed format outranks the queued kernels
    for (int64_t i = 0; i < n_iters; ++i) {
        thrml_moments* a = i + 1 == n_iters ? acc : nullptr;
        if (queue && (!a || observer_rides_along(a, s))) {
            s->pending.emplace_back(keys[i], a);
            if (s->pending.size() * static_cast<size_t>(s->prog->n_free) >= (s->sliced ? SLICE_MAX_STEPS : PERSIST_MAX_STEPS))
                if (int32_t rc = flush_pending(s)) return rc;
            continue;
        }
        if (int32_t rc = flush_pending(s)) return rc;
        if (int32_t rc = sweep(s, keys[i], inj, a)) return rc;
    }
    return THRML_OK;
}

int32_t thrml_sample_blocks(thrml_state* s, uint64_t key, const thrml_noise* inj) {
    if (!s) return fail(THRML_ERR_INVALID_ARG, "null state");
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    NoiseCursor nc;
    if (inj && inj->u) { nc.u = inj->u; nc.len = inj->len; }
    if (int32_t rc = sweep(s, key, nc.u ? &nc : nullptr)) return rc;
    CU_TRY(cudaStreamSynchronize(s->prog->ctx->stream));
    return check_err_flag(s);
}
int32_t thrml_run_blocks(thrml_state* s, uint64_t key, int64_t n_iters, const thrml_noise* inj) {
    if (!s) return fail(THRML_ERR_INVALID_ARG, "null state");
    if (n_iters < 0) return fail(THRML_ERR_INVALID_ARG, "n_iters must be non-negative");
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    s->pending.clear();  // sweeps queued by a call that failed half-way are not replayed
    NoiseCursor nc;
    if (inj && inj->u) { nc.u = inj->u; nc.len = inj->len; }
    if (int32_t rc = run(s, key, n_iters, nc.u ? &nc : nullptr)) return rc;
    if (int32_t rc = flush_pending(s)) return rc;
    CU_TRY(cudaStreamSynchronize(s->prog->ctx->stream));
    return check_err_flag(s);
}
// Device-to-device copy of one block's state between two states of the same program and chain count.
int32_t thrml_state_copy_block(thrml_state* dst, const thrml_state* src, int32_t block) {
    if (!dst || !src) return fail(THRML_ERR_INVALID_ARG, "null state");
    if (dst->prog != src->prog || dst->n_chains != src->n_chains) return fail(THRML_ERR_INVALID_ARG, "states must share the program and the chain count");
    if (int32_t rc = check_block(dst, block)) return rc;
    CU_TRY(cudaSetDevice(dst->device));
    const BlockProg& bp = dst->prog->blocks[block];
    cudaStream_t st = dst->prog->ctx->stream;
    CU_TRY(cudaMemcpyAsync(dst->rows(bp.sd) + bp.offset * dst->ld, src->rows(bp.sd) + bp.offset * src->ld, static_cast<size_t>(bp.n) * dst->ld, cudaMemcpyDeviceToDevice, st));
    dst->touch(block);
    if (dst->prog->is_dense_source[block]) {
        // A dense block reads this block as a +-1 bf16 image: the source state keeps its image (built once, it is a cache of
        // the bytes) and the copy carries it along with the per-node one counts, so the destination need not rebuild them.
        thrml_state* from = const_cast<thrml_state*>(src);
        if (int32_t rc = ensure_image(from, block, true)) return rc;
        if (int32_t rc = ensure_image(dst, block, false)) return rc;
        CU_TRY(cudaMemcpyAsync(dst->image[block]->p, from->image[block]->p, from->image[block]->bytes, cudaMemcpyDeviceToDevice, st));
        dst->image_fresh[block] = 1;
        if (from->ones_fresh[block] && from->ones[block]) {
            if (!dst->ones[block]) {
                dst->ones[block].reset(new DevBuf());
                if (int32_t rc = dst->ones[block]->alloc(static_cast<size_t>(bp.n) * 4)) return rc;
            }
            CU_TRY(cudaMemcpyAsync(dst->ones[block]->p, from->ones[block]->p, static_cast<size_t>(bp.n) * 4, cudaMemcpyDeviceToDevice, st));
            dst->ones_fresh[block] = 1;
        }
    }
    return THRML_OK;
}
int32_t thrml_ising_energy(thrml_state* s, int64_t n_nodes, const int64_t* nodes, const float* biases, int64_t n_edges, const int64_t* edges, const float* weights,
                           float beta, double* energy_out) {
    if (!s || !energy_out || n_nodes < 0 || n_edges < 0 || (n_nodes > 0 && (!nodes || !biases)) || (n_edges > 0 && (!edges || !weights)))
        return fail(THRML_ERR_INVALID_ARG, "bad energy arguments");
    thrml_program* p = s->prog;
    CU_TRY(cudaSetDevice(p->ctx->device));
    cudaStream_t st = p->ctx->stream;
    const int64_t n_terms = n_nodes + n_edges;
    std::vector<int32_t> pa(static_cast<size_t>(n_terms)), pb(static_cast<size_t>(n_terms));
    std::vector<float> w(static_cast<size_t>(n_terms));
    auto locate = [&](int64_t nd, int32_t* pos) -> int32_t {
        if (nd < 0 || nd >= static_cast<int64_t>(p->loc_sd.size()) || p->loc_sd[nd] < 0) return fail(THRML_ERR_INVALID_ARG, "Node not found in global location map");
        if (p->loc_sd[nd] != p->sd_spin) return fail(THRML_ERR_INVALID_ARG, "the Ising energy is defined on spin nodes");
        *pos = static_cast<int32_t>(p->loc_pos[nd]);
        return THRML_OK;
    };
    for (int64_t i = 0; i < n_nodes; ++i) {
        if (int32_t rc = locate(nodes[i], &pa[i])) return rc;
        pb[i] = -1;
        w[i] = biases[i];
    }
    for (int64_t e = 0; e < n_edges; ++e) {
        if (int32_t rc = locate(edges[2 * e], &pa[n_nodes + e])) return rc;
        if (int32_t rc = locate(edges[2 * e + 1], &pb[n_nodes + e])) return rc;
        w[n_nodes + e] = weights[e];
    }
    const int64_t n_chunks = std::max<int64_t>(1, (n_terms + ENERGY_CHUNK - 1) / ENERGY_CHUNK);
    DevBuf d_pa, d_pb, d_w, d_partial, d_out;
    if (int32_t rc = upload(d_pa, pa.data(), pa.size() * 4, st)) return rc;
    if (int32_t rc = upload(d_pb, pb.data(), pb.size() * 4, st)) return rc;
    if (int32_t rc = upload(d_w, w.data(), w.size() * 4, st)) return rc;
    if (int32_t rc = d_partial.alloc(static_cast<size_t>(n_chunks * s->ld) * 8)) return rc;
    if (int32_t rc = d_out.alloc(static_cast<size_t>(s->n_chains) * 8)) return rc;
    CU_TRY(cudaMemsetAsync(d_partial.p, 0, d_partial.bytes, st));
    if (n_terms > 0) {
        dim3 grid(static_cast<unsigned>(n_chunks), static_cast<unsigned>((s->ld / 4 + 31) / 32));
        k_energy_partial<<<grid, dim3(32, 8), 0, st>>>(d_pa.as<int32_t>(), d_pb.as<int32_t>(), d_w.as<float>(), n_terms, s->rows(p->sd_spin), s->ld, s->n_chains,
                                                       d_partial.as<double>());
        CU_TRY(cudaGetLastError());
    }
    k_energy_final<<<static_cast<unsigned>((s->n_chains + 255) / 256), 256, 0, st>>>(d_partial.as<double>(), n_chunks, s->ld, s->n_chains, -static_cast<double>(beta),
                                                                                     d_out.as<double>());
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaMemcpyAsync(energy_out, d_out.p, static_cast<size_t>(s->n_chains) * 8, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    return THRML_OK;
}

// DiscreteEBMFactor::factor_energy (discrete_ebm.rs:552-592) per chain; see the header for the argument layout.
int32_t thrml_factor_energy(thrml_state* s, int64_t rows, int32_t n_spin_groups, int32_t n_cat_groups, const int64_t* nodes, const float* w, int32_t d1, int32_t d2,
                            double* energy_out) {
    if (!s || !energy_out || rows < 0 || n_spin_groups < 0 || n_cat_groups < 0 || d1 < 1 || d2 < 1 || (rows > 0 && (!w || (n_spin_groups + n_cat_groups > 0 && !nodes))))
        return fail(THRML_ERR_INVALID_ARG, "bad factor energy arguments");
    if (n_cat_groups > 2) return fail(THRML_ERR_UNSUPPORTED, "weights are rank 3: at most two categorical node groups per factor");
    if ((n_cat_groups < 2 && d2 != 1) || (n_cat_groups < 1 && d1 != 1))
        return fail(THRML_ERR_INVALID_ARG, "The shape of the weight tensor must be [b, x_1, ..., x_k], where k is the length of categorical_node_groups");
    thrml_program* p = s->prog;
    CU_TRY(cudaSetDevice(p->ctx->device));
    cudaStream_t st = p->ctx->stream;
    const int32_t n_groups = n_spin_groups + n_cat_groups;
    std::vector<int32_t> pos(static_cast<size_t>(std::max<int64_t>(1, n_groups * rows)));
    for (int32_t g = 0; g < n_groups; ++g) {
        const int32_t want = g < n_spin_groups ? p->sd_spin : p->sd_cat;
        for (int64_t t = 0; t < rows; ++t) {
            const int64_t nd = nodes[g * rows + t];
            if (nd < 0 || nd >= static_cast<int64_t>(p->loc_sd.size()) || p->loc_sd[nd] < 0) return fail(THRML_ERR_INVALID_ARG, "Node not found in global location map");
            if (p->loc_sd[nd] != want) return fail(THRML_ERR_INVALID_ARG, "All nodes in a block must be of the same type: a spin group holds a categorical node or the reverse");
            pos[g * rows + t] = static_cast<int32_t>(p->loc_pos[nd]);
        }
    }
    const int64_t n_chunks = std::max<int64_t>(1, (rows + ENERGY_CHUNK - 1) / ENERGY_CHUNK);
    DevBuf d_pos, d_w, d_partial, d_out;
    if (int32_t rc = upload(d_pos, pos.data(), pos.size() * 4, st)) return rc;
    if (rows > 0)
        if (int32_t rc = upload(d_w, w, static_cast<size_t>(rows) * d1 * d2 * 4, st)) return rc;
    if (int32_t rc = d_partial.alloc(static_cast<size_t>(n_chunks * s->ld) * 8)) return rc;
    if (int32_t rc = d_out.alloc(static_cast<size_t>(s->n_chains) * 8)) return rc;
    CU_TRY(cudaMemsetAsync(d_partial.p, 0, d_partial.bytes, st));
    if (rows > 0) {
        dim3 grid(static_cast<unsigned>(n_chunks), static_cast<unsigned>((s->ld / 4 + 31) / 32));
        k_factor_energy_partial<<<grid, dim3(32, 8), 0, st>>>(d_pos.as<int32_t>(), n_spin_groups, n_cat_groups, d_w.as<float>(), d1, d2, rows,
                                                              p->sd_spin >= 0 ? s->rows(p->sd_spin) : nullptr, p->sd_cat >= 0 ? s->rows(p->sd_cat) : nullptr, s->ld,
                                                              d_partial.as<double>());
        CU_TRY(cudaGetLastError());
    }
    k_energy_final<<<static_cast<unsigned>((s->n_chains + 255) / 256), 256, 0, st>>>(d_partial.as<double>(), n_chunks, s->ld, s->n_chains, -1.0, d_out.as<double>());
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaMemcpyAsync(energy_out, d_out.p, static_cast<size_t>(s->n_chains) * 8, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    return THRML_OK;
}

// sample_single_block (program.rs:324-393): update one free block in place with the given block key.
int32_t thrml_sample_single_block(thrml_state* s, int32_t block, uint64_t key) {
    if (!s) return fail(THRML_ERR_INVALID_ARG, "null state");
    if (block < 0 || block >= s->prog->n_free) return fail(THRML_ERR_INVALID_ARG, "block index out of range");
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    const BlockProg& bp = s->prog->blocks[block];
    cudaStream_t st = s->prog->ctx->stream;
    if (s->prog->staged[bp.order]) {
        if (int32_t rc = launch_block(s, block, key, nullptr, s->stage.as<uint8_t>(), nullptr)) return rc;
        CU_TRY(cudaMemcpyAsync(s->rows(bp.sd) + bp.offset * s->ld, s->stage.p, static_cast<size_t>(bp.n) * s->ld, cudaMemcpyDeviceToDevice, st));
        s->touch(block);
    } else if (int32_t rc = launch_block(s, block, key, nullptr, s->rows(bp.sd) + bp.offset * s->ld, nullptr)) {
        return rc;
    }
    CU_TRY(cudaStreamSynchronize(st));
    return check_err_flag(s);
}

// <s_a s_b> over this device's chains for every node pair of two spin blocks, on the tensor cores (asynchronous; result in
// s->d_corr as f32 [n_a][n_b]).
// `a_from` (nullable): another state of the same program and chain count that supplies block a.
static int32_t pair_correlation_async(thrml_state* s, int32_t block_a, int32_t block_b, float* d_out, thrml_state* a_from = nullptr) {
    thrml_program* p = s->prog;
    auto state_of = [&](int32_t blk) -> thrml_state* { return a_from && blk == block_a ? a_from : s; };
    if (p->blocks[block_a].is_cat || p->blocks[block_b].is_cat) return fail(THRML_ERR_INVALID_ARG, "pair correlations are defined for spin blocks");
    cudaStream_t st = p->ctx->stream;
    if (int32_t rc = ensure_err_flag(s)) return rc;
    // Rows of the GEMM come from block a unless only block b fills 256-row pair tiles well: then the operands swap
    // and the epilogue writes the transposed result, which lands in the same [n_a][n_b] layout.
    bool pair = use_pair_tiles(p->dense_tiles, p->blocks[block_a].n, s->n_chains), swapped = false;
    if (!pair && p->dense_tiles == 2 && use_pair_tiles(2, p->blocks[block_b].n, s->n_chains)) pair = swapped = true;
    const int32_t row_block = swapped ? block_b : block_a, col_block = swapped ? block_a : block_b;
    const BlockProg& br = p->blocks[row_block];
    const BlockProg& bc = p->blocks[col_block];
    CUtensorMap map_a, map_b;  // encoded per call: kernel parameters are copied at launch
    if (int32_t rc = make_operand_map(&map_a, state_of(row_block)->rows(br.sd) + br.offset * s->ld, true, s->n_chains, br.n, s->ld, dense::BM)) return rc;
    const int bn = pair ? pair_tile_width(bc.n) : (bc.n >= 2048 ? 256 : 64);
    if (int32_t rc = make_operand_map(&map_b, state_of(col_block)->rows(bc.sd) + bc.offset * s->ld, true, s->n_chains, bc.n, s->ld, pair ? bn / 2 : bn)) return rc;
    for (int32_t blk : {block_a, block_b}) {
        const BlockProg& bp = p->blocks[blk];
        thrml_state* o = state_of(blk);
        if (o->ones_fresh.empty()) return fail(THRML_ERR_INVALID_ARG, "state without block bookkeeping");
        if (!o->ones[blk]) {
            o->ones[blk].reset(new DevBuf());
            if (int32_t rc = o->ones[blk]->alloc(static_cast<size_t>(bp.n) * 4)) return rc;
        }
        if (!o->ones_fresh[blk]) {
            dense::k_row_ones<<<static_cast<unsigned>((bp.n + 7) / 8), dim3(32, 8), 0, st>>>(o->rows(bp.sd) + bp.offset * o->ld, o->ld, o->n_chains, static_cast<int32_t>(bp.n),
                                                                                             o->ones[blk]->as<int32_t>());
            CU_TRY(cudaGetLastError());
            o->ones_fresh[blk] = 1;
        }
    }
    dense::GemmArgs g{};
    g.m_total = static_cast<int32_t>(br.n);
    g.n_total = static_cast<int32_t>(bc.n);
    g.k_bytes = static_cast<int32_t>(s->n_chains);
    g.ones_a = state_of(row_block)->ones[row_block]->as<int32_t>();
    g.ones_b = state_of(col_block)->ones[col_block]->as<int32_t>();
    g.corr_out = d_out;
    g.corr_transposed = swapped ? 1 : 0;
    g.n_chains = static_cast<int32_t>(s->n_chains);
    if (pair) {
        if (bn == 256) return launch_dense_pair<dense::EPI_CORR, 256>(s, map_a, map_b, g);
        if (bn == 208) return launch_dense_pair<dense::EPI_CORR, 208>(s, map_a, map_b, g);
        return launch_dense_pair<dense::EPI_CORR, 128>(s, map_a, map_b, g);
    }
    if (bn == 256) return launch_dense<dense::EPI_CORR, 256>(s, map_a, map_b, g);
    return launch_dense<dense::EPI_CORR, 64>(s, map_a, map_b, g);
}
int32_t thrml_pair_correlation(thrml_state* s, int32_t block_a, int32_t block_b, float* host_out) {
    if (!s || !host_out) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (int32_t rc = check_block(s, block_a)) return rc;
    if (int32_t rc = check_block(s, block_b)) return rc;
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    const size_t cnt = static_cast<size_t>(s->prog->blocks[block_a].n) * s->prog->blocks[block_b].n;
    if (!s->d_corr.holds(2 * cnt * 4))
        if (int32_t rc = s->d_corr.alloc(2 * cnt * 4)) return rc;
    if (int32_t rc = pair_correlation_async(s, block_a, block_b, s->d_corr.as<float>())) return rc;
    CU_TRY(cudaMemcpyAsync(host_out, s->d_corr.p, cnt * 4, cudaMemcpyDeviceToHost, s->prog->ctx->stream));
    CU_TRY(cudaStreamSynchronize(s->prog->ctx->stream));
    return check_err_flag(s);
}
// One contrastive-divergence step on a two-layer model: load the visible data, h0 ~ P(h | v0), positive correlations
// <v0 h0>, one Gibbs sweep (sample_blocks), negative correlations <v1 h1>.
int32_t thrml_cd1_step(thrml_state* s, int32_t visible_block, int32_t hidden_block, const uint8_t* v0_host, uint64_t key, float* pos_host, float* neg_host) {
    if (!s) return fail(THRML_ERR_INVALID_ARG, "null state");
    if (visible_block < 0 || visible_block >= s->prog->n_free || hidden_block < 0 || hidden_block >= s->prog->n_free || visible_block == hidden_block)
        return fail(THRML_ERR_INVALID_ARG, "visible and hidden must be two distinct free blocks");
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    cudaStream_t st = s->prog->ctx->stream;
    const size_t cnt = static_cast<size_t>(s->prog->blocks[visible_block].n) * s->prog->blocks[hidden_block].n;
    if (!s->d_corr.holds(2 * cnt * 4))
        if (int32_t rc = s->d_corr.alloc(2 * cnt * 4)) return rc;
    if (v0_host)
        if (int32_t rc = thrml_state_upload_u8(s, visible_block, v0_host)) return rc;
    uint64_t keys[2];
    rng_split(key, 2, keys);
    const BlockProg& hb = s->prog->blocks[hidden_block];
    if (int32_t rc = launch_block(s, hidden_block, keys[0], nullptr, s->rows(hb.sd) + hb.offset * s->ld, nullptr)) return rc;
    if (int32_t rc = pair_correlation_async(s, visible_block, hidden_block, s->d_corr.as<float>())) return rc;
    s->no_image_block = hidden_block;  // h1 feeds only the correlations, which read the byte state
    const int32_t rc_sweep = sweep(s, keys[1], nullptr);
    s->no_image_block = -1;
    if (rc_sweep) return rc_sweep;
    if (int32_t rc = pair_correlation_async(s, visible_block, hidden_block, s->d_corr.as<float>() + cnt)) return rc;
    if (pos_host) CU_TRY(cudaMemcpyAsync(pos_host, s->d_corr.p, cnt * 4, cudaMemcpyDeviceToHost, st));
    if (neg_host) CU_TRY(cudaMemcpyAsync(neg_host, s->d_corr.as<float>() + cnt, cnt * 4, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    return check_err_flag(s);
}

// The same step with the visible data read from another state of the program (`data`, same chain count) instead of being
// copied in first: h0 ~ P(h | data's visible block) and <v0 h0> read `data`; the sweep then writes v1 and h1 into `s`, whose
// own visible block is never read before it is overwritten.  `data` is not modified (its cached +-1 image and one counts
// are built on first use).
__global__ void k_scale_f32(float* x, int64_t n, float f) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) x[i] = __fmul_rn(x[i], f);
}
static int32_t cd1_step_from(thrml_state* s, thrml_state* data, int32_t visible_block, int32_t hidden_block, uint64_t key, thrml_comm* comm, float* pos_host, float* neg_host);
int32_t thrml_cd1_step_from(thrml_state* s, thrml_state* data, int32_t visible_block, int32_t hidden_block, uint64_t key, float* pos_host, float* neg_host) {
    return cd1_step_from(s, data, visible_block, hidden_block, key, nullptr, pos_host, neg_host);
}
// Chains sharded over the ranks of `comm` (each rank its own data and chain states, global chain ids through the states'
// chain offsets): the two correlation matrices are means over a rank's chains; one ncclAllReduce adds them and
// a scale by 1 / ranks makes them the means over all chains (exact when the chain count per rank is a power of two).
int32_t thrml_cd1_step_comm(thrml_state* s, thrml_state* data, int32_t visible_block, int32_t hidden_block, uint64_t key, thrml_comm* comm, float* pos_host,
                            float* neg_host) {
    if (!comm) return fail(THRML_ERR_INVALID_ARG, "null communicator");
    if (s && comm->ctx != s->prog->ctx) return fail(THRML_ERR_INVALID_ARG, "communicator and state belong to different contexts");
    return cd1_step_from(s, data, visible_block, hidden_block, key, comm, pos_host, neg_host);
}
static int32_t cd1_step_from(thrml_state* s, thrml_state* data, int32_t visible_block, int32_t hidden_block, uint64_t key, thrml_comm* comm, float* pos_host, float* neg_host) {
    if (!s || !data) return fail(THRML_ERR_INVALID_ARG, "null state");
    if (comm && s == data) return fail(THRML_ERR_INVALID_ARG, "the sharded step reads its data from a second state");
    if (s == data) return thrml_cd1_step(s, visible_block, hidden_block, nullptr, key, pos_host, neg_host);
    if (s->prog != data->prog || s->n_chains != data->n_chains) return fail(THRML_ERR_INVALID_ARG, "states must share the program and the chain count");
    if (visible_block < 0 || visible_block >= s->prog->n_free || hidden_block < 0 || hidden_block >= s->prog->n_free || visible_block == hidden_block)
        return fail(THRML_ERR_INVALID_ARG, "visible and hidden must be two distinct free blocks");
    const BlockProg& hb = s->prog->blocks[hidden_block];
    if (hb.kernel != 3 || hb.dense_src != visible_block) {  // not on the dense path: bring the data over and run the ordinary step
        if (comm) return fail(THRML_ERR_UNSUPPORTED, "the sharded CD-1 step needs the hidden block on the dense path");
        if (int32_t rc = thrml_state_copy_block(s, data, visible_block)) return rc;
        return thrml_cd1_step(s, visible_block, hidden_block, nullptr, key, pos_host, neg_host);
    }
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    cudaStream_t st = s->prog->ctx->stream;
    const size_t cnt = static_cast<size_t>(s->prog->blocks[visible_block].n) * hb.n;
    if (!s->d_corr.holds(2 * cnt * 4))
        if (int32_t rc = s->d_corr.alloc(2 * cnt * 4)) return rc;
    uint64_t keys[2];
    rng_split(key, 2, keys);
    ++s->block_launches;
    if (int32_t rc = dense_update(s, hidden_block, static_cast<uint32_t>(keys[0]), static_cast<uint32_t>(keys[0] >> 32), data)) return rc;
    if (int32_t rc = pair_correlation_async(s, visible_block, hidden_block, s->d_corr.as<float>(), data)) return rc;
    s->no_image_block = hidden_block;  // h1 feeds only the correlations, which read the byte state
    const int32_t rc_sweep = sweep(s, keys[1], nullptr);
    s->no_image_block = -1;
    if (rc_sweep) return rc_sweep;
    if (int32_t rc = pair_correlation_async(s, visible_block, hidden_block, s->d_corr.as<float>() + cnt)) return rc;
    if (comm && comm->world > 1) {
        const NcclApi* api = nccl_api();
        if (!api) return fail(THRML_ERR_NCCL, "NCCL is not available");
        NCCL_TRY(api, AllReduce(s->d_corr.p, s->d_corr.p, 2 * cnt, ncclFloat32, ncclSum, comm->nccl, st));
        k_scale_f32<<<static_cast<unsigned>((2 * cnt + 255) / 256), 256, 0, st>>>(s->d_corr.as<float>(), static_cast<int64_t>(2 * cnt), 1.0f / static_cast<float>(comm->world));
        CU_TRY(cudaGetLastError());
    }
    if (pos_host) CU_TRY(cudaMemcpyAsync(pos_host, s->d_corr.p, cnt * 4, cudaMemcpyDeviceToHost, st));
    if (neg_host) CU_TRY(cudaMemcpyAsync(neg_host, s->d_corr.as<float>() + cnt, cnt * 4, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    return check_err_flag(s);
}

// Failure-detection self test: one warp waits, with the same bounded wait the tensor-core pipeline uses, on a barrier
// nothing ever arrives on.  The wait runs out, the kernel raises its error flag and returns, and the host reports
// THRML_ERR_TIMEOUT; the context stays usable.
__global__ void k_wait_on_nothing(int* err, uint32_t* polls) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        dense::mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool ok = dense::mbar_wait(&bar, 0, err, 7);
        *polls = ok ? 0u : 1u;
    }
}
int32_t thrml_debug_wait_timeout(thrml_ctx* ctx) {
    if (!ctx) return fail(THRML_ERR_INVALID_ARG, "null context");
    CU_TRY(cudaSetDevice(ctx->device));
    DevBuf flag;
    if (int32_t rc = flag.alloc(8)) return rc;
    CU_TRY(cudaMemsetAsync(flag.p, 0, 8, ctx->stream));
    k_wait_on_nothing<<<1, 32, 0, ctx->stream>>>(flag.as<int>(), flag.as<uint32_t>() + 1);
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaStreamSynchronize(ctx->stream));
    int host[2] = {0, 0};
    CU_TRY(cudaMemcpy(host, flag.p, 8, cudaMemcpyDeviceToHost));
    if (host[0] != 0) return fail(THRML_ERR_TIMEOUT, "a bounded wait ran out (role " + std::to_string(host[0]) + "); the kernel returned and the context is intact");
    return THRML_OK;
}

int32_t thrml_fields_debug(thrml_state* s, int32_t block, float* out) {
    if (!s || !out) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (block < 0 || block >= s->prog->n_free) return fail(THRML_ERR_INVALID_ARG, "block index out of range");
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    const BlockProg& bp = s->prog->blocks[block];
    const size_t cnt = static_cast<size_t>(bp.n) * s->n_chains * (bp.is_cat ? bp.kind : 1);
    DevBuf tmp;
    if (int32_t rc = tmp.alloc(cnt * 4)) return rc;
    if (bp.kernel == 3) {  // a block on the dense path reports the fields its tensor-core kernel draws from
        if (int32_t rc = dense_fields(s, block, tmp.as<float>())) return rc;
    } else if (int32_t rc = launch_block(s, block, 0, nullptr, nullptr, tmp.as<float>())) {
        return rc;
    }
    CU_TRY(cudaMemcpyAsync(out, tmp.p, cnt * 4, cudaMemcpyDeviceToHost, s->prog->ctx->stream));
    CU_TRY(cudaStreamSynchronize(s->prog->ctx->stream));
    return check_err_flag(s);
}

// ---------------------------------------------------------------------------------------------------------
// Observers.
// ---------------------------------------------------------------------------------------------------------
int32_t thrml_moments_create(thrml_program* p, int32_t n_types, const int64_t* rows_per_type, const int64_t* row_ptr, const int64_t* members,
                             int32_t transform_to_spin, thrml_moments** out) {
    if (!p || !out || n_types < 0 || (n_types > 0 && (!rows_per_type || !row_ptr))) return fail(THRML_ERR_INVALID_ARG, "bad moment spec");
    CU_TRY(cudaSetDevice(p->ctx->device));
    auto m = std::make_unique<thrml_moments>();
    m->prog = p;
    m->device = p->device;
    m->kernel_epoch = p->kernel_epoch;
    m->spin_transform = transform_to_spin ? 1 : 0;
    m->rows_per_type.assign(rows_per_type, rows_per_type + n_types);
    for (int64_t r : m->rows_per_type) {
        if (r < 0) return fail(THRML_ERR_INVALID_ARG, "negative row count");
        m->total_rows += r;
    }
    const int64_t n_mem = m->total_rows ? row_ptr[m->total_rows] : 0;
    std::vector<int32_t> sd(static_cast<size_t>(n_mem)), pos(static_cast<size_t>(n_mem));
    for (int64_t q = 0; q < n_mem; ++q) {
        const int64_t nd = members[q];
        if (nd < 0 || nd >= static_cast<int64_t>(p->loc_sd.size()) || p->loc_sd[nd] < 0) return fail(THRML_ERR_INVALID_ARG, "Node not found in global location map");
        sd[q] = p->loc_sd[nd];
        pos[q] = static_cast<int32_t>(p->loc_pos[nd]);
    }
    cudaStream_t st = p->ctx->stream;
    const int64_t zero = 0;
    // Split the rows: single spins and neighbour pairs of threshold-table blocks are accumulated by the update kernel
    // itself; every other row (clamped nodes, other kernels, longer tuples, repeated rows, raw products) goes to k_moments.
    {
        std::vector<std::vector<int32_t>> m1(p->n_free), m2(p->n_free);
        std::vector<int32_t> block_of_pos;  // spin class only
        if (p->sd_spin >= 0) {
            block_of_pos.assign(static_cast<size_t>(p->class_size[p->sd_spin]), -1);
            for (size_t bi = 0; bi < p->blocks.size(); ++bi)
                if (!p->blocks[bi].is_cat)
                    for (int64_t j = 0; j < p->blocks[bi].n; ++j) block_of_pos[p->blocks[bi].offset + j] = static_cast<int32_t>(bi);
        }
        // blocks whose update kernel can carry the observer: threshold-table (8 slots per node) and sequential-sum (32)
        auto lut_block = [&](int32_t bi) {
            return bi >= 0 && bi < p->n_free && (p->blocks[bi].kernel == 1 || p->blocks[bi].kernel == 4 || p->blocks[bi].kernel == 6);
        };
        auto slots_of = [&](int32_t bi) { return p->blocks[bi].kernel == 1 ? LUT_BITS : SEQ_MAX; };
        auto is_hub = [&](int32_t bi, int64_t i) { return !p->blocks[bi].h_hub.empty() && p->blocks[bi].h_hub[static_cast<size_t>(i)] != 0; };
        for (int32_t bi = 0; bi < p->n_free; ++bi)
            if (lut_block(bi)) {
                m1[bi].assign(static_cast<size_t>(p->blocks[bi].n), -1);
                m2[bi].assign(static_cast<size_t>(p->blocks[bi].n) * slots_of(bi), -1);
            }
        std::vector<int64_t> left_ptr(1, 0), left_rows;
        std::vector<int32_t> left_sd, left_pos;
        for (int64_t r = 0; r < m->total_rows; ++r) {
            const int64_t b0 = row_ptr[r], len = row_ptr[r + 1] - b0;
            bool taken = false;
            if (m->spin_transform && len == 1 && sd[b0] == p->sd_spin) {
                const int32_t bi = block_of_pos[pos[b0]];
                if (lut_block(bi) && !is_hub(bi, pos[b0] - p->blocks[bi].offset)) {
                    int32_t& slot = m1[bi][pos[b0] - p->blocks[bi].offset];
                    if (slot < 0) { slot = static_cast<int32_t>(r); taken = true; }
                }
            } else if (m->spin_transform && len == 2 && sd[b0] == p->sd_spin && sd[b0 + 1] == p->sd_spin && r <= 0x7fffffff) {
                int32_t pa = pos[b0], pb = pos[b0 + 1];
                int32_t ba = block_of_pos[pa], bb = block_of_pos[pb];
                if (p->blocks[ba].order < p->blocks[bb].order) { std::swap(pa, pb); std::swap(ba, bb); }  // (pa, ba) is updated later
                if (p->blocks[ba].order > p->blocks[bb].order && lut_block(ba) && !is_hub(ba, pa - p->blocks[ba].offset)) {
                    const int64_t i = pa - p->blocks[ba].offset;
                    const int ns = slots_of(ba);
                    for (int j = 0; j < ns; ++j)
                        if (p->blocks[ba].h_nbr[i * ns + j] == pb && m2[ba][i * ns + j] < 0) {
                            m2[ba][i * ns + j] = static_cast<int32_t>(r);
                            taken = true;
                            break;
                        }
                }
            }
            if (taken) { m->any_fused = true; continue; }
            for (int64_t q = b0; q < b0 + len; ++q) { left_sd.push_back(sd[q]); left_pos.push_back(pos[q]); }
            left_ptr.push_back(static_cast<int64_t>(left_sd.size()));
            left_rows.push_back(r);
        }
        m->n_left = static_cast<int64_t>(left_rows.size());
        m->fused.resize(p->n_free);
        if (m->any_fused) {
            for (int32_t bi = 0; bi < p->n_free; ++bi) {
                if (!lut_block(bi)) continue;
                m->fused[bi].reset(new FusedMaps());
                if (int32_t rc = upload(m->fused[bi]->m1, m1[bi].data(), m1[bi].size() * 4, st)) return rc;
                if (int32_t rc = upload(m->fused[bi]->m2, m2[bi].data(), m2[bi].size() * 4, st)) return rc;
            }
            if (int32_t rc = upload(m->d_left_ptr, left_ptr.data(), left_ptr.size() * 8, st)) return rc;
            if (int32_t rc = upload(m->d_left_sd, left_sd.data(), left_sd.size() * 4, st)) return rc;
            if (int32_t rc = upload(m->d_left_pos, left_pos.data(), left_pos.size() * 4, st)) return rc;
            if (int32_t rc = upload(m->d_left_rows, left_rows.data(), left_rows.size() * 8, st)) return rc;
            CU_TRY(cudaStreamSynchronize(st));
            m->left_all_spin = m->spin_transform && p->sd_spin >= 0 && std::all_of(left_sd.begin(), left_sd.end(), [&](int32_t c) { return c == p->sd_spin; });
        }
    }
    m->all_spin = m->spin_transform && p->sd_spin >= 0 && std::all_of(sd.begin(), sd.end(), [&](int32_t c) { return c == p->sd_spin; });
    if (int32_t rc = upload(m->d_row_ptr, m->total_rows ? row_ptr : &zero, static_cast<size_t>(m->total_rows + 1) * 8, st)) return rc;
    if (int32_t rc = upload(m->d_mem_sd, sd.data(), sd.size() * 4, st)) return rc;
    if (int32_t rc = upload(m->d_mem_pos, pos.data(), pos.size() * 4, st)) return rc;
    if (int32_t rc = m->d_sums.alloc(static_cast<size_t>(m->sum_slots() + 2) * 8)) return rc;
    CU_TRY(cudaMemsetAsync(m->d_sums.p, 0, m->d_sums.bytes, st));
    CU_TRY(cudaStreamSynchronize(st));
    *out = m.release();
    return THRML_OK;
}
int32_t thrml_marginals_create(thrml_program* p, const int32_t* blocks, int32_t n_blocks, int32_t K, thrml_moments** out) {
    if (!p || !out || !blocks || n_blocks <= 0 || K < 1 || K > 255) return fail(THRML_ERR_INVALID_ARG, "bad marginal spec");
    CU_TRY(cudaSetDevice(p->ctx->device));
    auto m = std::make_unique<thrml_moments>();
    m->prog = p;
    m->device = p->device;
    m->mode = 1;
    m->K = K;
    std::vector<int32_t> sd, pos;
    for (int32_t i = 0; i < n_blocks; ++i) {
        if (blocks[i] < 0 || blocks[i] >= p->n_free + p->n_clamped) return fail(THRML_ERR_INVALID_ARG, "block index out of range");
        const BlockProg& bp = p->blocks[blocks[i]];
        for (int64_t j = 0; j < bp.n; ++j) {
            sd.push_back(bp.sd);
            pos.push_back(static_cast<int32_t>(bp.offset + j));
        }
    }
    m->total_rows = static_cast<int64_t>(sd.size()) * K;
    m->rows_per_type.assign(1, m->total_rows);
    cudaStream_t st = p->ctx->stream;
    if (int32_t rc = upload(m->d_node_sd, sd.data(), sd.size() * 4, st)) return rc;
    if (int32_t rc = upload(m->d_node_pos, pos.data(), pos.size() * 4, st)) return rc;
    if (int32_t rc = m->d_sums.alloc(static_cast<size_t>(m->sum_slots() + 2) * 8)) return rc;
    CU_TRY(cudaMemsetAsync(m->d_sums.p, 0, m->d_sums.bytes, st));
    CU_TRY(cudaStreamSynchronize(st));
    *out = m.release();
    return THRML_OK;
}
void thrml_moments_destroy(thrml_moments* m) {
    if (!m) return;
    cudaSetDevice(m->device);
    cudaDeviceSynchronize();
    delete m;
}
int32_t thrml_moments_reset(thrml_moments* m) {
    if (!m) return fail(THRML_ERR_INVALID_ARG, "null moments");
    CU_TRY(cudaSetDevice(m->prog->ctx->device));
    CU_TRY(cudaMemsetAsync(m->d_sums.p, 0, m->d_sums.bytes, m->prog->ctx->stream));
    CU_TRY(cudaStreamSynchronize(m->prog->ctx->stream));
    m->n_obs = 0;
    return THRML_OK;
}
static int32_t observe_async(thrml_moments* m, thrml_state* s) {
    if (m->prog != s->prog) return fail(THRML_ERR_INVALID_ARG, "observer and state belong to different programs");
    if (int32_t rc = flush_pending(s)) return rc;
    cudaStream_t st = s->prog->ctx->stream;
    const uint8_t* c0 = s->rows(0);
    const uint8_t* c1 = s->rows(1);
    if (m->mode == 0) {
        if (m->total_rows > 0) {
            const unsigned grid = static_cast<unsigned>((m->total_rows + 7) / 8);
            if (m->all_spin)
                k_moments_spin<<<grid, dim3(32, 8), 0, st>>>(m->d_row_ptr.as<int64_t>(), m->d_mem_pos.as<int32_t>(), m->total_rows, s->rows(s->prog->sd_spin), s->ld, s->n_chains,
                                                             m->d_sums.as<unsigned long long>(), nullptr);
            else
                k_moments<<<grid, dim3(32, 8), 0, st>>>(m->d_row_ptr.as<int64_t>(), m->d_mem_sd.as<int32_t>(), m->d_mem_pos.as<int32_t>(), m->total_rows, c0, c1, s->ld,
                                                        s->n_chains, m->spin_transform, m->d_sums.as<unsigned long long>(), nullptr);
            CU_TRY(cudaGetLastError());
        }
    } else {
        const int64_t nodes = m->total_rows / m->K;
        k_marginals<<<static_cast<unsigned>((nodes + 7) / 8), dim3(32, 8), 0, st>>>(m->d_node_sd.as<int32_t>(), m->d_node_pos.as<int32_t>(), nodes, m->K, c0, c1, s->ld,
                                                                                     s->n_chains, m->d_sums.as<unsigned long long>());
        CU_TRY(cudaGetLastError());
    }
    m->n_obs += s->n_chains;
    return THRML_OK;
}
int32_t thrml_moments_observe(thrml_moments* m, thrml_state* s) {
    if (!m || !s) return fail(THRML_ERR_INVALID_ARG, "null argument");
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    if (int32_t rc = observe_async(m, s)) return rc;
    CU_TRY(cudaStreamSynchronize(s->prog->ctx->stream));
    return THRML_OK;
}
int32_t thrml_moments_read(thrml_moments* m, int32_t type, int64_t* sums_out, int64_t* n_obs_out) {
    if (!m) return fail(THRML_ERR_INVALID_ARG, "null moments");
    if (type < 0 || type >= static_cast<int32_t>(m->rows_per_type.size())) return fail(THRML_ERR_INVALID_ARG, "moment type out of range");
    CU_TRY(cudaSetDevice(m->prog->ctx->device));
    int64_t start = 0;
    for (int32_t t = 0; t < type; ++t) start += m->rows_per_type[t];
    if (sums_out && m->rows_per_type[type] > 0) {
        CU_TRY(cudaMemcpyAsync(sums_out, m->d_sums.as<int64_t>() + start, static_cast<size_t>(m->rows_per_type[type]) * 8, cudaMemcpyDeviceToHost, m->prog->ctx->stream));
        CU_TRY(cudaStreamSynchronize(m->prog->ctx->stream));
    }
    if (n_obs_out) *n_obs_out = m->n_obs;
    return THRML_OK;
}
int32_t thrml_moments_device_buffer(thrml_moments* m, void** dev_ptr_out, int64_t* count_out) {
    if (!m) return fail(THRML_ERR_INVALID_ARG, "null moments");
    if (dev_ptr_out) *dev_ptr_out = m->d_sums.p;
    if (count_out) *count_out = m->total_rows;
    return THRML_OK;
}
// The one collective of the chain-parallel path: sums (and the observation count) added over the ranks of `comm`, in
// place on every rank.  Two tiny reductions first agree on the total and the largest per-rank observation count; when
// no total can leave 32 bits the sums travel as int32 (half the bytes), else as int64.  Every rank takes the same branch
// because the decision uses only reduced values.
int32_t thrml_moments_allreduce(thrml_moments* m, thrml_comm* comm) {
    if (!m || !comm) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (comm->ctx != m->prog->ctx) return fail(THRML_ERR_INVALID_ARG, "communicator and observer belong to different contexts");
    if (comm->world == 1) return THRML_OK;
    const NcclApi* api = nccl_api();
    if (!api) return THRML_ERR_NCCL;
    CU_TRY(cudaSetDevice(m->device));
    cudaStream_t st = m->prog->ctx->stream;
    long long* sums = m->d_sums.as<long long>();
    long long* slots = sums + m->sum_slots();
    const long long mine[2] = {m->n_obs, m->n_obs};
    CU_TRY(cudaMemcpyAsync(slots, mine, sizeof(mine), cudaMemcpyHostToDevice, st));
    NCCL_TRY(api, GroupStart());
    NCCL_TRY(api, AllReduce(slots, slots, 1, ncclInt64, ncclSum, comm->nccl, st));
    NCCL_TRY(api, AllReduce(slots + 1, slots + 1, 1, ncclInt64, ncclMax, comm->nccl, st));
    NCCL_TRY(api, GroupEnd());
    long long got[2] = {0, 0};
    CU_TRY(cudaMemcpyAsync(got, slots, sizeof(got), cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    const int64_t rows = m->total_rows;
    if (rows > 0) {
        // |sum| of a row on one rank <= that rank's observation count (products of +-1, or category counts)
        const bool fits32 = (m->spin_transform || m->mode == 1) && got[1] * static_cast<long long>(comm->world) < (1LL << 31);
        if (fits32) {
            if (int32_t rc = m->d_narrow.reserve(static_cast<size_t>(rows) * 4)) return rc;
            const unsigned grid = static_cast<unsigned>((rows + 255) / 256);
            k_narrow_i64<<<grid, 256, 0, st>>>(sums, m->d_narrow.as<int32_t>(), rows);
            CU_TRY(cudaGetLastError());
            NCCL_TRY(api, AllReduce(m->d_narrow.p, m->d_narrow.p, static_cast<size_t>(rows), ncclInt32, ncclSum, comm->nccl, st));
            k_widen_i32<<<grid, 256, 0, st>>>(m->d_narrow.as<int32_t>(), sums, rows);
            CU_TRY(cudaGetLastError());
        } else {
            NCCL_TRY(api, AllReduce(sums, sums, static_cast<size_t>(rows), ncclInt64, ncclSum, comm->nccl, st));
        }
    }
    m->n_obs = got[0];
    return THRML_OK;
}
int32_t thrml_moments_fused_info(const thrml_moments* m, int64_t* n_fused_rows, int64_t* n_other_rows) {
    if (!m) return fail(THRML_ERR_INVALID_ARG, "null moments");
    const int64_t other = m->any_fused ? m->n_left : m->total_rows;
    if (n_fused_rows) *n_fused_rows = m->total_rows - other;
    if (n_other_rows) *n_other_rows = other;
    return THRML_OK;
}
int32_t thrml_program_set_option(thrml_program* p, int32_t option, double value) {
    if (!p) return fail(THRML_ERR_INVALID_ARG, "null program");
    if (option == THRML_OPT_DENSE_TILES) {
        if (value != 0.0 && value != 1.0 && value != 2.0) return fail(THRML_ERR_INVALID_ARG, "dense tiles: 0 (one CTA per tile), 1 (CTA pairs) or 2 (per launch)");
        p->dense_tiles = static_cast<int32_t>(value);
        return THRML_OK;
    }
    if (option == THRML_OPT_SPLIT_MARGIN) {
        if (!(value >= 0.0)) return fail(THRML_ERR_INVALID_ARG, "the split margin is a non-negative number of 2^-24 units");
        p->split_extra_margin = static_cast<float>(value);
        CU_TRY(cudaSetDevice(p->device));
        for (int32_t bi = 0; bi < p->n_free; ++bi)
            if (p->blocks[bi].n_split > 0)
                if (int32_t rc = rebuild_seq(p, p->blocks[bi])) return rc;
        CU_TRY(cudaStreamSynchronize(p->ctx->stream));
        return THRML_OK;
    }
    if (option == THRML_OPT_STATE_FORMAT) {
        if (value != 0.0 && value != 1.0) return fail(THRML_ERR_INVALID_ARG, "state format: 0 (one byte per spin) or 1 (bit-packed mirror)");
        p->state_format = static_cast<int32_t>(value);
        return THRML_OK;
    }
    if (option == THRML_OPT_GATHER_ONLY) {
        if (value != 0.0 && value != 1.0) return fail(THRML_ERR_INVALID_ARG, "gather only: 0 or 1");
        p->gather_only = value != 0.0;
        return THRML_OK;
    }
    return fail(THRML_ERR_INVALID_ARG, "unknown program option " + std::to_string(option));
}
int32_t thrml_program_get_option(const thrml_program* p, int32_t option, double* value_out) {
    if (!p || !value_out) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (option == THRML_OPT_DENSE_TILES) *value_out = p->dense_tiles;
    else if (option == THRML_OPT_SPLIT_MARGIN) *value_out = p->split_extra_margin;
    else if (option == THRML_OPT_GATHER_ONLY) *value_out = p->gather_only ? 1.0 : 0.0;
    else if (option == THRML_OPT_STATE_FORMAT) *value_out = p->state_format;
    else return fail(THRML_ERR_INVALID_ARG, "unknown program option " + std::to_string(option));
    return THRML_OK;
}
// Bring-up check of the CTA-pair kernels: both CTAs of a pair must have been given the same tensor-memory base address
// (the two-CTA MMA writes both accumulators at one address).  Reads the two words the last pair launch recorded.
int32_t thrml_debug_pair_tmem_check(thrml_state* s) {
    if (!s) return fail(THRML_ERR_INVALID_ARG, "null state");
    if (!s->d_dense_debug.p) return THRML_OK;  // no tensor-core kernel has run on this state
    CU_TRY(cudaSetDevice(s->device));
    CU_TRY(cudaStreamSynchronize(s->prog->ctx->stream));
    uint32_t base[2] = {0, 0};
    CU_TRY(cudaMemcpy(base, s->d_dense_debug.p, sizeof(base), cudaMemcpyDeviceToHost));
    if (base[0] != base[1])
        return fail(THRML_ERR_CUDA, "the two CTAs of a pair got different tensor-memory addresses (" + std::to_string(base[0]) + ", " + std::to_string(base[1]) + ")");
    return THRML_OK;
}
int32_t thrml_state_launch_counts(const thrml_state* s, int64_t* block_launches, int64_t* persistent_launches) {
    if (!s) return fail(THRML_ERR_INVALID_ARG, "null state");
    if (block_launches) *block_launches = s->block_launches;
    if (persistent_launches) *persistent_launches = s->persistent_launches;
    return THRML_OK;
}
int32_t thrml_moments_add_observations(thrml_moments* m, int64_t n_obs) {
    if (!m) return fail(THRML_ERR_INVALID_ARG, "null moments");
    m->n_obs += n_obs;
    return THRML_OK;
}

// StateObserver (state_observer.rs:25-47): copy the listed blocks' rows, [observed node][chain].
static int32_t observe_states(thrml_state* s, const int32_t* obs_blocks, int32_t n_obs_blocks, uint8_t* dst) {
    if (int32_t rc = flush_pending(s)) return rc;
    cudaStream_t st = s->prog->ctx->stream;
    int64_t row = 0;
    for (int32_t i = 0; i < n_obs_blocks; ++i) {
        const BlockProg& bp = s->prog->blocks[obs_blocks[i]];
        CU_TRY(cudaMemcpy2DAsync(dst + row * s->n_chains, static_cast<size_t>(s->n_chains), s->rows(bp.sd) + bp.offset * s->ld, static_cast<size_t>(s->ld),
                                 static_cast<size_t>(s->n_chains), static_cast<size_t>(bp.n), cudaMemcpyDeviceToHost, st));
        row += bp.n;
    }
    return THRML_OK;
}

int32_t thrml_sample_with_observation(thrml_state* s, uint64_t key, int64_t n_warmup, int64_t n_samples, int64_t steps_per_sample, thrml_moments* moments,
                                      const int32_t* obs_blocks, int32_t n_obs_blocks, uint8_t* obs_out, const thrml_noise* inj) {
    if (!s) return fail(THRML_ERR_INVALID_ARG, "null state");
    if (n_warmup < 0 || n_samples < 0 || steps_per_sample < 0) return fail(THRML_ERR_INVALID_ARG, "schedule entries must be non-negative");
    if (obs_out && (!obs_blocks || n_obs_blocks <= 0)) return fail(THRML_ERR_INVALID_ARG, "obs_out needs a block list");
    CU_TRY(cudaSetDevice(s->prog->ctx->device));
    s->pending.clear();
    int64_t obs_rows = 0;
    for (int32_t i = 0; i < n_obs_blocks; ++i) {
        if (int32_t rc = check_block(s, obs_blocks[i])) return rc;
        obs_rows += s->prog->blocks[obs_blocks[i]].n;
    }
    NoiseCursor nc;
    if (inj && inj->u) { nc.u = inj->u; nc.len = inj->len; }
    NoiseCursor* ncp = nc.u ? &nc : nullptr;
    uint64_t two[2];
    rng_split(key, 2, two);  // split_two, sampling.rs:189
    if (moments && moments->prog != s->prog) return fail(THRML_ERR_INVALID_ARG, "observer and state belong to different programs");
    if (int32_t rc = run(s, two[0], n_warmup, ncp, moments)) return rc;
    if (obs_out)
        if (int32_t rc = observe_states(s, obs_blocks, n_obs_blocks, obs_out)) return rc;
    if (n_samples > 1) {  // sampling.rs:215-217,249-257: nothing more for n_samples <= 1
        std::vector<uint64_t> keys(static_cast<size_t>(n_samples - 1));
        rng_split(two[1], n_samples - 1, keys.data());
        const int64_t stride = obs_rows * s->n_chains;
        for (int64_t i = 0; i < n_samples - 1; ++i) {
            if (int32_t rc = run(s, keys[i], steps_per_sample, ncp, moments)) return rc;
            if (obs_out)
                if (int32_t rc = observe_states(s, obs_blocks, n_obs_blocks, obs_out + (i + 1) * stride)) return rc;
        }
    }
    if (int32_t rc = flush_pending(s)) return rc;
    CU_TRY(cudaStreamSynchronize(s->prog->ctx->stream));
    return check_err_flag(s);
}

// grad[r] = -beta (sum_pos[r] / denom_pos - sum_neg[r] / denom_neg), the means rounded to f32 first as estimate_moments
// returns them (ising.rs:489-502, 589-591).
__global__ void k_kl_grad(const long long* pos, const long long* neg, double denom_pos, double denom_neg, float neg_beta, int64_t n, float* out) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float mp = static_cast<float>(static_cast<double>(pos[i]) / denom_pos), mn = static_cast<float>(static_cast<double>(neg[i]) / denom_neg);
    out[i] = __fmul_rn(__fsub_rn(mp, mn), neg_beta);
}
// estimate_kl_grad (ising.rs:531-594): both phases and the gradient on the device; see the header.
int32_t thrml_estimate_kl_grad(thrml_state* pos, thrml_state* neg, thrml_moments* moments_pos, thrml_moments* moments_neg, uint64_t key, int64_t warmup_pos,
                               int64_t samples_pos, int64_t steps_pos, int64_t warmup_neg, int64_t samples_neg, int64_t steps_neg, float beta, float* grad_w_out,
                               float* grad_b_out) {
    if (!pos || !neg || !moments_pos || !moments_neg) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (moments_pos->prog != pos->prog || moments_neg->prog != neg->prog) return fail(THRML_ERR_INVALID_ARG, "each observer must belong to its phase's program");
    if (pos->prog->ctx != neg->prog->ctx) return fail(THRML_ERR_INVALID_ARG, "both phases must run on one context");
    if (moments_pos->mode != 0 || moments_neg->mode != 0 || moments_pos->rows_per_type != moments_neg->rows_per_type || moments_pos->rows_per_type.size() != 2)
        return fail(THRML_ERR_INVALID_ARG, "both observers must hold the same two moment types: bias nodes, then weight edges (ising_moment_spec)");
    if (samples_pos < 1 || samples_neg < 1) return fail(THRML_ERR_INVALID_ARG, "each phase needs at least one sample");
    uint64_t two[2];
    rng_split(key, 2, two);  // key.split_two(), ising.rs:543
    if (int32_t rc = thrml_moments_reset(moments_pos)) return rc;
    if (int32_t rc = thrml_moments_reset(moments_neg)) return rc;
    if (int32_t rc = thrml_sample_with_observation(pos, two[0], warmup_pos, samples_pos, steps_pos, moments_pos, nullptr, 0, nullptr, nullptr)) return rc;
    if (int32_t rc = thrml_sample_with_observation(neg, two[1], warmup_neg, samples_neg, steps_neg, moments_neg, nullptr, 0, nullptr, nullptr)) return rc;
    cudaStream_t st = pos->prog->ctx->stream;
    CU_TRY(cudaSetDevice(pos->device));
    const int64_t n_b = moments_pos->rows_per_type[0], n_w = moments_pos->rows_per_type[1], total = n_b + n_w;
    if (total == 0) return THRML_OK;
    DevBuf d_grad;
    if (int32_t rc = d_grad.alloc(static_cast<size_t>(total) * 4)) return rc;
    // estimate_moments divides by n_samples (ising.rs:489-502); a batch of chains is averaged as well
    k_kl_grad<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(moments_pos->d_sums.as<long long>(), moments_neg->d_sums.as<long long>(),
                                                                        static_cast<double>(moments_pos->n_obs), static_cast<double>(moments_neg->n_obs), -beta, total,
                                                                        d_grad.as<float>());
    CU_TRY(cudaGetLastError());
    if (grad_b_out && n_b > 0) CU_TRY(cudaMemcpyAsync(grad_b_out, d_grad.p, static_cast<size_t>(n_b) * 4, cudaMemcpyDeviceToHost, st));
    if (grad_w_out && n_w > 0) CU_TRY(cudaMemcpyAsync(grad_w_out, d_grad.as<float>() + n_b, static_cast<size_t>(n_w) * 4, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    return THRML_OK;
}

// sample_states (sampling.rs:128-156) with the samples streamed to the host bit-packed: bits_out[sample][observed node][word],
// word w holds chains 32w..32w+31 (bit c & 31).  Spin blocks only.  Samples are packed on the device into a staging
// buffer and copied out in chunks, so the host link carries one bit per spin instead of one byte (or the reference's f32).
int32_t thrml_sample_states_packed(thrml_state* s, uint64_t key, int64_t n_warmup, int64_t n_samples, int64_t steps_per_sample, const int32_t* obs_blocks,
                                   int32_t n_obs_blocks, uint32_t* bits_out) {
    if (!s || !obs_blocks || n_obs_blocks <= 0 || !bits_out) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (n_warmup < 0 || n_samples < 0 || steps_per_sample < 0) return fail(THRML_ERR_INVALID_ARG, "schedule entries must be non-negative");
    thrml_program* p = s->prog;
    CU_TRY(cudaSetDevice(p->ctx->device));
    s->pending.clear();
    cudaStream_t st = p->ctx->stream;
    int64_t rows = 0;
    for (int32_t i = 0; i < n_obs_blocks; ++i) {
        if (int32_t rc = check_block(s, obs_blocks[i])) return rc;
        if (p->blocks[obs_blocks[i]].is_cat) return fail(THRML_ERR_UNSUPPORTED, "bit-packed streaming is for spin blocks");
        rows += p->blocks[obs_blocks[i]].n;
    }
    const int64_t words = (s->n_chains + 31) / 32;
    const int64_t per_sample = rows * words;  // u32 per sample
    const int64_t total_samples = std::max<int64_t>(n_samples, 1);
    const int64_t chunk = std::max<int64_t>(1, std::min<int64_t>(total_samples, (int64_t(64) << 20) / std::max<int64_t>(per_sample * 4, 1)));
    DevBuf stage;
    if (int32_t rc = stage.alloc(static_cast<size_t>(chunk * per_sample) * 4)) return rc;
    int64_t in_chunk = 0, flushed = 0;
    auto pack = [&]() -> int32_t {
        if (int32_t rc = flush_pending(s)) return rc;
        uint32_t* dst = stage.as<uint32_t>() + in_chunk * per_sample;
        int64_t row = 0;
        for (int32_t i = 0; i < n_obs_blocks; ++i) {
            const BlockProg& bp = p->blocks[obs_blocks[i]];
            k_pack_rows<<<static_cast<unsigned>((bp.n + 7) / 8), dim3(32, 8), 0, st>>>(s->rows(bp.sd) + bp.offset * s->ld, s->ld, s->n_chains, bp.n, words, dst + row * words);
            CU_TRY(cudaGetLastError());
            row += bp.n;
        }
        if (++in_chunk == chunk) {
            CU_TRY(cudaMemcpyAsync(bits_out + flushed * per_sample, stage.p, static_cast<size_t>(in_chunk * per_sample) * 4, cudaMemcpyDeviceToHost, st));
            CU_TRY(cudaStreamSynchronize(st));  // the staging buffer is reused by the next chunk
            flushed += in_chunk;
            in_chunk = 0;
        }
        return THRML_OK;
    };
    uint64_t two[2];
    rng_split(key, 2, two);
    if (int32_t rc = run(s, two[0], n_warmup, nullptr)) return rc;
    if (int32_t rc = pack()) return rc;
    if (n_samples > 1) {
        std::vector<uint64_t> keys(static_cast<size_t>(n_samples - 1));
        rng_split(two[1], n_samples - 1, keys.data());
        for (int64_t i = 0; i < n_samples - 1; ++i) {
            if (int32_t rc = run(s, keys[i], steps_per_sample, nullptr)) return rc;
            if (int32_t rc = pack()) return rc;
        }
    }
    if (in_chunk > 0) CU_TRY(cudaMemcpyAsync(bits_out + flushed * per_sample, stage.p, static_cast<size_t>(in_chunk * per_sample) * 4, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    return check_err_flag(s);
}

}  // extern "C"
