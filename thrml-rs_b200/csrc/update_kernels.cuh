// Block-update kernels: generic spin and categorical updates for any slot-table structure, the threshold-table spin
// update (one launch per block), and its two multi-sweep variants for small programs.
//
// State layout: one byte per node and chain, chains innermost: state[class][global position][ld], ld = chains rounded
// up to 16 bytes.  A neighbour gather therefore reads one contiguous row segment per neighbour, whatever the graph.
#pragma once
#include <cooperative_groups.h>
#include <cstdint>
#include <cuda_runtime.h>

#include "device_math.cuh"

using namespace thrml;

constexpr int MAX_TAILS = 8;
constexpr int LUT_BITS = 8;              // a threshold table covers at most 8 neighbour spins
constexpr int LUT_SIZE = 1 << LUT_BITS;  // entries per node
constexpr int NARROW_CHUNKS = 4;         // up to 64 chains: blocks of the sequential-sum kinds run the node x quad gather kernel
constexpr int FEW_CHAIN_CHUNKS = 16;     // up to 16 chunks of 16 chains (256 chains): the thread-per-node threshold-table kernel

// Device view of one slot table.
struct DevTable {
    int32_t k, wdim, n_spin, n_tails;
    const int32_t* idx[MAX_TAILS];
    const uint8_t* active;
    const float* w;
};

struct UpdateArgs {
    const DevTable* tabs;
    int32_t n_tabs;
    int32_t n;            // nodes in the block
    int32_t K;            // categories (categorical kernel)
    int64_t ld;           // bytes per state row
    int64_t n_chains;
    uint32_t chain_word0; // global chain id of local chain 0, divided by 4
    const uint8_t* spin;  // class rows (may be null when the class is absent)
    const uint8_t* cat;
    uint8_t* dst;         // first row of the block's output (state rows or staging rows)
    uint32_t k0, k1;      // block key
    const float* inj;     // injected uniforms or null
    float* fields;        // debug output or null
};

__device__ __forceinline__ uint32_t ld_word(const uint8_t* base, int64_t row, int64_t ld, int quad) {
    return *reinterpret_cast<const uint32_t*>(base + row * ld + 4 * static_cast<int64_t>(quad));
}

// Generic spin update: any number of tables, spin tails and one optional categorical tail per table.
// One thread = one node x four consecutive chains.  MODE 0 in-kernel noise, 1 injected noise, 2 write gamma only.
// Field accumulation order: per table, slots left to right from zero; tables left to right (spin_gibbs.rs:527-582).
template <int MODE>
__global__ void __launch_bounds__(256) k_spin_generic(UpdateArgs a) {
    const int quad = blockIdx.y * blockDim.x + threadIdx.x;
    const int node = blockIdx.x * blockDim.y + threadIdx.y;
    if (node >= a.n || 4 * static_cast<int64_t>(quad) >= a.ld) return;
    float gamma[4] = {0.f, 0.f, 0.f, 0.f};
    for (int t = 0; t < a.n_tabs; ++t) {
        const DevTable T = a.tabs[t];
        float gs[4] = {0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < T.k; ++j) {
            const int64_t flat = static_cast<int64_t>(node) * T.k + j;
            if (!T.active[flat]) continue;
            float sp[4] = {1.f, 1.f, 1.f, 1.f};
            for (int tl = 0; tl < T.n_spin; ++tl) {
                const uint32_t wd = ld_word(a.spin, T.idx[tl][flat], a.ld, quad);
#pragma unroll
                for (int c = 0; c < 4; ++c) sp[c] = __fmul_rn(sp[c], ((wd >> (8 * c)) & 1u) ? 1.0f : -1.0f);
            }
            if (T.n_tails > T.n_spin) {  // first categorical tail selects the weight (spin_gibbs.rs:556-577)
                const uint32_t wd = ld_word(a.cat, T.idx[T.n_spin][flat], a.ld, quad);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t x = (wd >> (8 * c)) & 0xffu;
                    const float wv = x < static_cast<uint32_t>(T.wdim) ? T.w[flat * T.wdim + x] : 0.0f;
                    gs[c] = __fadd_rn(gs[c], __fmul_rn(wv, sp[c]));
                }
            } else {
                const float wv = T.w[flat * T.wdim];
#pragma unroll
                for (int c = 0; c < 4; ++c) gs[c] = __fadd_rn(gs[c], __fmul_rn(wv, sp[c]));
            }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) gamma[c] = __fadd_rn(gamma[c], gs[c]);
    }
    if (MODE == 2) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int64_t chain = 4 * static_cast<int64_t>(quad) + c;
            if (chain < a.n_chains) a.fields[chain * a.n + node] = gamma[c];
        }
        return;
    }
    U4 r{0, 0, 0, 0};
    if (MODE == 0) r = philox4x32_10(static_cast<uint32_t>(node), a.chain_word0 + static_cast<uint32_t>(quad), 0u, TAG_SPIN, a.k0, a.k1);
    uint32_t out = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int64_t chain = 4 * static_cast<int64_t>(quad) + c;
        float u;
        if (MODE == 1) u = chain < a.n_chains ? a.inj[static_cast<int64_t>(node) * a.n_chains + chain] : 2.0f;
        else u = u24(pick(r, c));
        const float p = det_sigmoid(__fmul_rn(gamma[c], 2.0f));  // spin_gibbs.rs:95
        if (u <= p && chain < a.n_chains) out |= 1u << (8 * c);   // spin_gibbs.rs:97
    }
    *reinterpret_cast<uint32_t*>(a.dst + static_cast<int64_t>(node) * a.ld + 4 * static_cast<int64_t>(quad)) = out;
}

// Generic categorical update (softmax.rs:586-709 + 60-97): logits theta[c] = sum over tables and slots of
// active * prod(2s-1) * W[own c, neighbour category]; draw = argmax_c(theta[c] - ln(-ln u_c)), first maximum wins.
template <int MODE>
__global__ void __launch_bounds__(256) k_cat_generic(UpdateArgs a) {
    const int quad = blockIdx.y * blockDim.x + threadIdx.x;
    const int node = blockIdx.x * blockDim.y + threadIdx.y;
    if (node >= a.n || 4 * static_cast<int64_t>(quad) >= a.ld) return;
    const int K = a.K;
    float best[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t arg[4] = {0, 0, 0, 0};
    U4 r[4];
    for (int cat = 0; cat < K; ++cat) {
        float th[4] = {0.f, 0.f, 0.f, 0.f};
        for (int t = 0; t < a.n_tabs; ++t) {
            const DevTable T = a.tabs[t];
            const bool has_cat = T.n_tails > T.n_spin;
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < T.k; ++j) {
                const int64_t flat = static_cast<int64_t>(node) * T.k + j;
                if (!T.active[flat]) continue;
                float sp[4] = {1.f, 1.f, 1.f, 1.f};
                for (int tl = 0; tl < T.n_spin; ++tl) {
                    const uint32_t wd = ld_word(a.spin, T.idx[tl][flat], a.ld, quad);
#pragma unroll
                    for (int c = 0; c < 4; ++c) sp[c] = __fmul_rn(sp[c], ((wd >> (8 * c)) & 1u) ? 1.0f : -1.0f);
                }
                if (has_cat) {
                    const uint32_t wd = ld_word(a.cat, T.idx[T.n_spin][flat], a.ld, quad);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t x = (wd >> (8 * c)) & 0xffu;
                        if (x >= static_cast<uint32_t>(K)) x = K - 1;
                        sum[c] = __fadd_rn(sum[c], __fmul_rn(sp[c], T.w[flat * T.wdim + cat * K + x]));
                    }
                } else {
                    const float wv = T.w[flat * T.wdim + cat];
#pragma unroll
                    for (int c = 0; c < 4; ++c) sum[c] = __fadd_rn(sum[c], __fmul_rn(sp[c], wv));
                }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) th[c] = __fadd_rn(th[c], sum[c]);
        }
        if (MODE == 2) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int64_t chain = 4 * static_cast<int64_t>(quad) + c;
                if (chain < a.n_chains) a.fields[(chain * a.n + node) * K + cat] = th[c];
            }
        }
#pragma unroll
        for (int c = 0; MODE != 2 && c < 4; ++c) {  // no draws in the fields-only instantiation
            const int64_t chain = 4 * static_cast<int64_t>(quad) + c;
            float u;
            if (MODE == 1) {
                u = chain < a.n_chains ? a.inj[(static_cast<int64_t>(node) * K + cat) * a.n_chains + chain] : 0.5f;
            } else {
                if ((cat & 3) == 0)
                    r[c] = philox4x32_10(static_cast<uint32_t>(node), 4u * (a.chain_word0 + static_cast<uint32_t>(quad)) + c, static_cast<uint32_t>(cat >> 2), TAG_CAT, a.k0, a.k1);
                u = u23_open(pick(r[c], cat & 3));
            }
            const float g = -det_log(-det_log(u));  // softmax.rs:84
            const float p = __fadd_rn(th[c], g);
            if (cat == 0 || p > best[c]) {  // strict >: the first maximum wins (gumbel_argmax/kernel.rs:81-83)
                best[c] = p;
                arg[c] = cat;
            }
        }
    }
    if (MODE == 2) return;
    uint32_t out = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c)
        if (4 * static_cast<int64_t>(quad) + c < a.n_chains) out |= arg[c] << (8 * c);
    *reinterpret_cast<uint32_t*>(a.dst + static_cast<int64_t>(node) * a.ld + 4 * static_cast<int64_t>(quad)) = out;
}

// Exact Gumbel-argmax of ONE chain of a categorical node, the generic way (softmax.rs:586-709, 60-97).  Out of line:
// k_cat_fast calls it for the rare draws whose two best categories its fast logarithms cannot separate.
__device__ __noinline__ uint32_t cat_exact_argmax(const UpdateArgs& a, int node, int quad, int c) {
    const int K = a.K;
    const int sh = 8 * c;
    float best = 0.f;
    uint32_t arg = 0;
    U4 r{0, 0, 0, 0};
    for (int cat = 0; cat < K; ++cat) {
        float th = 0.f;
        for (int t = 0; t < a.n_tabs; ++t) {
            const DevTable& T = a.tabs[t];
            const bool has_cat = T.n_tails > T.n_spin;
            float sum = 0.f;
            for (int j = 0; j < T.k; ++j) {
                const int64_t flat = static_cast<int64_t>(node) * T.k + j;
                if (!T.active[flat]) continue;
                float sp = 1.f;
                for (int tl = 0; tl < T.n_spin; ++tl) sp = __fmul_rn(sp, ((ld_word(a.spin, T.idx[tl][flat], a.ld, quad) >> sh) & 1u) ? 1.0f : -1.0f);
                float wv;
                if (has_cat) {
                    uint32_t x = (ld_word(a.cat, T.idx[T.n_spin][flat], a.ld, quad) >> sh) & 0xffu;
                    if (x >= static_cast<uint32_t>(K)) x = K - 1;
                    wv = T.w[flat * T.wdim + cat * K + x];
                } else {
                    wv = T.w[flat * T.wdim + cat];
                }
                sum = __fadd_rn(sum, __fmul_rn(sp, wv));
            }
            th = __fadd_rn(th, sum);
        }
        if ((cat & 3) == 0)
            r = philox4x32_10(static_cast<uint32_t>(node), 4u * (a.chain_word0 + static_cast<uint32_t>(quad)) + c, static_cast<uint32_t>(cat >> 2), TAG_CAT, a.k0, a.k1);
        const float p = __fadd_rn(th, -det_log(-det_log(u23_open(pick(r, cat & 3)))));
        if (cat == 0 || p > best) { best = p; arg = cat; }
    }
    return arg;
}

// Categorical update for blocks whose nodes have at most CAT_SLOTS active slots (in-kernel noise only; more would not fit the register file).  Same results
// as k_cat_generic<0>, organised for speed (with 128 chains or more a warp is one node, so the slot structure is warp-uniform).
//  * everything that does not depend on the category is gathered once per node and thread: per active slot the
//    neighbour's category word (clamped), the sign word of its spin tails, the weight row and whether it opens a table;
//  * the category loop then costs one table lookup and one add per slot and chain, in the canonical order
//    (per table from zero, tables left to right);
//  * the Gumbel noise is screened with the hardware logarithm (k_potts_update documents the bound: each score within
//    2e-5 of the exact one); a leader less than 6e-5 ahead of the runner-up sends that chain to cat_exact_argmax.
//  * STAGE: the threads of a node (they share a warp) first copy the node's weight rows into shared memory — K x K floats
//    per slot, coalesced — so the lookups of the category loop are shared-memory reads instead of dependent global
//    gathers (the launch picks it when CAT_SLOTS x K x K floats per node of the CTA fit in 48 KiB).
constexpr int CAT_SLOTS = 8;
template <bool STAGE>
__global__ void __launch_bounds__(256, 4) k_cat_fast(const __grid_constant__ UpdateArgs a) {
    extern __shared__ float s_w[];  // STAGE: [blockDim.y][CAT_SLOTS][K * K]
    const int quad = blockIdx.y * blockDim.x + threadIdx.x;
    const int node = blockIdx.x * blockDim.y + threadIdx.y;
    const bool valid = node < a.n && 4 * static_cast<int64_t>(quad) < a.ld;
    const bool walks = STAGE ? node < a.n : valid;  // STAGE: every thread of a live node helps to copy its weights
    if (!STAGE && !valid) return;
    const int K = a.K;
    float* mine = s_w + static_cast<size_t>(threadIdx.y) * CAT_SLOTS * K * K;
    uint32_t xw[CAT_SLOTS], sg[CAT_SLOTS];   // neighbour categories (4 chains), sign bits (bit 7 of a byte: the spin-tail product is -1)
    const float* wrow[CAT_SLOTS];            // weights of the slot: [K][K] with a categorical tail, [K] without
    uint32_t opens = 0, tailed = 0;          // bit s: slot s opens a table / has a categorical tail
    int S = 0;
    // One active slot: its neighbour words, sign word, weight row (and the copy of its weights) under the static index S.
    auto take_slot = [&](const DevTable& T, int64_t flat, bool first, int at) {
        uint32_t neg = 0;
        for (int tl = 0; tl < (valid ? T.n_spin : 0); ++tl) neg ^= ~ld_word(a.spin, T.idx[tl][flat], a.ld, quad);
        uint32_t x = 0;
        if (valid && T.n_tails > T.n_spin) {
            x = ld_word(a.cat, T.idx[T.n_spin][flat], a.ld, quad);
            x = __vminu4(x, static_cast<uint32_t>(K - 1) * 0x01010101u);  // per-byte clamp, as the generic kernel does
        }
#pragma unroll
        for (int s = 0; s < CAT_SLOTS; ++s)
            if (s == at) {  // static indices keep the lists in registers
                xw[s] = x;
                sg[s] = (neg & 0x01010101u) << 7;
                wrow[s] = T.w + flat * T.wdim;
            }
        if (STAGE) {  // the node's threads copy the slot's weights: every thread of the node walks the same slots
            const int len = T.n_tails > T.n_spin ? K * K : K;
            const float* src = T.w + flat * T.wdim;
            for (int i = threadIdx.x; i < len; i += blockDim.x) mine[at * K * K + i] = __ldg(src + i);
        }
        if (first) opens |= 1u << at;
        if (T.n_tails > T.n_spin) tailed |= 1u << at;
    };
    // Which slots are active.  With a warp per node (128 chains or more) lane L looks at candidate L of the node's
    // (table, slot) list, one ballot gives the active ones in the canonical order, and the per-slot loads below are
    // independent of each other; walking the tables slot by slot instead makes every load wait for the previous flag.
    bool listed = false;
    if (STAGE && blockDim.x == 32) {
        int ct = -1, cj = 0, total = 0;
        for (int t = 0; t < a.n_tabs; ++t) {
            const int k = a.tabs[t].k;
            if (static_cast<int>(threadIdx.x) >= total && static_cast<int>(threadIdx.x) < total + k) {
                ct = t;
                cj = static_cast<int>(threadIdx.x) - total;
            }
            total += k;
        }
        if (total <= 32) {  // uniform over the CTA
            listed = true;
            bool act = false;
            if (walks && ct >= 0) act = a.tabs[ct].active[static_cast<int64_t>(node) * a.tabs[ct].k + cj] != 0;
            const uint32_t mask = __ballot_sync(0xffffffffu, act);
            const int n_act = min(__popc(mask), CAT_SLOTS);
            int t_prev = -1;
#pragma unroll
            for (int s = 0; s < CAT_SLOTS; ++s) {
                const uint32_t src = __fns(mask, 0, s + 1) & 31u;
                const int ts = __shfl_sync(0xffffffffu, ct, static_cast<int>(src)), js = __shfl_sync(0xffffffffu, cj, static_cast<int>(src));
                if (s < n_act) {  // uniform over the warp
                    const DevTable& T = a.tabs[ts];
                    take_slot(T, static_cast<int64_t>(node) * T.k + js, ts != t_prev, s);
                    t_prev = ts;
                }
            }
            S = n_act;
        }
    }
    if (!listed) {
        for (int t = 0; t < (walks ? a.n_tabs : 0); ++t) {
            const DevTable& T = a.tabs[t];
            bool first = true;
            for (int j = 0; j < T.k; ++j) {
                const int64_t flat = static_cast<int64_t>(node) * T.k + j;
                if (!T.active[flat]) continue;
                take_slot(T, flat, first, S);
                ++S;
                first = false;
            }
        }
    }
    if (STAGE) {
        __syncwarp();  // a node's threads lie in one warp (blockDim.x divides 32)
        if (!valid) return;
    }
    constexpr float MARGIN = 1.2e-5f;
    uint32_t out = 0;
    // One chain at a time (not unrolled): the four chains of a thread share nothing in this loop but the slot data, and the
    // smaller live set (one Philox block, one leader / runner-up pair) lets three CTAs share an SM instead of two.
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
        if (4 * static_cast<int64_t>(quad) + c >= a.n_chains) break;
        const int sh = 8 * c;
        float best = 0.f, second = -3.0e38f, lmin = 1.0f;
        uint32_t lead = 0;
        U4 r{0, 0, 0, 0};
        for (int cat = 0; cat < K; ++cat) {
            float th = 0.f, sum = 0.f;
#pragma unroll
            for (int s = 0; s < CAT_SLOTS; ++s) {
                if (s >= S) break;  // uniform over the threads of a node
                if (s > 0 && ((opens >> s) & 1u)) { th = __fadd_rn(th, sum); sum = 0.f; }
                uint32_t wb;
                if (STAGE) {
                    wb = __float_as_uint(mine[s * K * K + (((tailed >> s) & 1u) ? cat * K + ((xw[s] >> sh) & 0xffu) : cat)]);
                } else {
                    const float* wk = ((tailed >> s) & 1u) ? wrow[s] + cat * K + ((xw[s] >> sh) & 0xffu) : wrow[s] + cat;
                    wb = __float_as_uint(__ldg(wk));
                }
                sum = __fadd_rn(sum, __uint_as_float(wb ^ (((sg[s] >> sh) & 0x80u) << 24)));  // sp * w = w with the sign flipped
            }
            th = __fadd_rn(th, sum);
            if ((cat & 3) == 0)
                r = philox4x32_10(static_cast<uint32_t>(node), 4u * (a.chain_word0 + static_cast<uint32_t>(quad)) + c, static_cast<uint32_t>(cat >> 2), TAG_CAT, a.k0, a.k1);
            // the 23-bit uniform (m + 0.5) 2^-23 of u23_open, formed exactly as (1 + m 2^-23) - (1 - 2^-24)
            const float u = __uint_as_float(0x3f800000u | (pick(r, cat & 3) >> 9)) - 0.99999994039535522461f;
            const float l1 = lg2_normal(u) * -0.6931471805599453f;            // -ln u > 0
            const float p = fmaf(lg2_normal(l1), -0.6931471805599453f, th);  // th - ln(l1)
            if (cat == 0) {
                best = p;
                lmin = l1;
            } else {
                lmin = fminf(lmin, l1);
                second = fmaxf(second, fminf(best, p));
                if (p > best) { best = p; lead = cat; }
            }
        }
        // The hardware logarithm's absolute error (1.7e-7 in ln u) is a relative error of 1.7e-7 / l in l = -ln u and so an
        // absolute error of that size in ln l; the outer logarithm and the final add stay below 4e-6.  A leader more than
        // three such bounds ahead (taken at the chain's smallest l) is the exact argmax; anything closer is recomputed exactly.
        if (!(best - second > MARGIN + 6.0e-7f * rcp_normal(lmin))) lead = cat_exact_argmax(a, node, quad, c);
        out |= lead << sh;
    }
    *reinterpret_cast<uint32_t*>(a.dst + static_cast<int64_t>(node) * a.ld + 4 * static_cast<int64_t>(quad)) = out;
}

// Warp-per-node form of k_cat_fast for K <= 16 and 128 chains or more: same states, a quarter of its instructions.
//  * a warp owns a node for ALL chains: it stages the node's weight rows in shared memory once (a slot with a categorical
//    tail transposed to [neighbour category][own category], rows padded to a multiple of four floats) and then walks the
//    chains 128 at a time, instead of one CTA per 128 chains staging the same weights again;
//  * the logits of one chain live in registers (th[KT]): per slot the row of the neighbour's category is fetched with
//    16-byte shared-memory loads and added with the sign of the spin tails, so a slot costs about three instructions per
//    category instead of twenty (no per-category slot bookkeeping, no address arithmetic);
//  * the canonical order is kept: a table's slots are summed from zero and the table sums are added left to right (a
//    table with a single active slot adds its weight directly: 0 + w = w);
//  * entry lists (table and slot of the node's active slots) come from the host, as for k_spin_wide;
//  * noise, screen and exact fallback are k_cat_fast's.
struct CatWarpArgs {
    UpdateArgs u;
    const int32_t* ent;     // [n][CAT_SLOTS]: table << 24 | slot, -1 = none
    const uint32_t* first;  // [n] bit e: entry e opens a table
    const int32_t* cnt;     // [n]
    int32_t n_chunks4;      // ld / 4: four-chain words per state row
    PhiloxRoundKeys rk;
};
template <int KT>
__global__ void __launch_bounds__(256, 3) k_cat_warp(const __grid_constant__ CatWarpArgs a) {
    extern __shared__ float4 s_w4[];  // [8 warps][CAT_SLOTS][K][KP], KP = K rounded up to a multiple of 4
    constexpr int NV = (KT + 3) / 4;
    constexpr float MARGIN = 1.2e-5f;
    const int lane = threadIdx.x & 31;
    const int K = a.u.K;
    const int KP = (K + 3) & ~3;
    float* mine = reinterpret_cast<float*>(s_w4) + static_cast<size_t>(threadIdx.x >> 5) * CAT_SLOTS * K * KP;
    for (int node = blockIdx.x * 8 + (threadIdx.x >> 5); node < a.u.n; node += gridDim.x * 8) {
        const int cnt = __ldg(a.cnt + node);
        const uint32_t first = __ldg(a.first + node);
        const uint32_t opens_mask = first, closes_mask = cnt > 0 ? ((first >> 1) | (1u << (cnt - 1))) : 0u;  // slot s closes its table when s + 1 opens one or s is the last
        // lane e < cnt: entry e's tail positions and weight row
        int32_t nb0 = -1, nb1 = -1, nb2 = -1, nbc = -1;
        const float* wp = nullptr;
        if (lane < cnt) {
            const int32_t code = __ldg(a.ent + static_cast<int64_t>(node) * CAT_SLOTS + lane);
            const DevTable& T = a.u.tabs[code >> 24];
            const int64_t flat = static_cast<int64_t>(node) * T.k + (code & 0xffffff);
            if (T.n_spin > 0) nb0 = __ldg(T.idx[0] + flat);
            if (T.n_spin > 1) nb1 = __ldg(T.idx[1] + flat);
            if (T.n_spin > 2) nb2 = __ldg(T.idx[2] + flat);
            if (T.n_tails > T.n_spin) nbc = __ldg(T.idx[T.n_spin] + flat);
            wp = T.w + flat * T.wdim;
        }
        const uint32_t tailed = __ballot_sync(0xffffffffu, nbc >= 0);
        __syncwarp();  // the previous node's lookups are done
        for (int s = 0; s < cnt; ++s) {
            const float* src = reinterpret_cast<const float*>(__shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(wp), s));
            float* dst = mine + s * K * KP;
            if ((tailed >> s) & 1u) {
                for (int i = lane; i < K * K; i += 32) {
                    const int own = i / K, x = i - own * K;
                    dst[x * KP + own] = __ldg(src + i);
                }
            } else {
                for (int i = lane; i < K; i += 32) dst[i] = __ldg(src + i);
            }
        }
        __syncwarp();
        uint8_t* drow = a.u.dst + static_cast<int64_t>(node) * a.u.ld;
        for (int base = 0; base < a.n_chunks4; base += 32) {  // every lane runs every pass: the entry broadcasts are warp-wide
            const int quad = base + lane;
            const bool live = quad < a.n_chunks4;
            uint32_t xw[CAT_SLOTS], sg[CAT_SLOTS];  // neighbour categories of 4 chains (clamped); bit 0 of a byte: the spin-tail product is -1
#pragma unroll
            for (int s = 0; s < CAT_SLOTS; ++s) {
                xw[s] = sg[s] = 0;
                if (s < cnt) {  // uniform over the warp
                    const int32_t n0 = __shfl_sync(0xffffffffu, nb0, s), n1 = __shfl_sync(0xffffffffu, nb1, s), n2 = __shfl_sync(0xffffffffu, nb2, s);
                    const int32_t nc = __shfl_sync(0xffffffffu, nbc, s);
                    if (live) {
                        uint32_t neg = 0;
                        if (n0 >= 0) neg ^= ~ld_word(a.u.spin, n0, a.u.ld, quad);
                        if (n1 >= 0) neg ^= ~ld_word(a.u.spin, n1, a.u.ld, quad);
                        if (n2 >= 0) neg ^= ~ld_word(a.u.spin, n2, a.u.ld, quad);
                        sg[s] = neg & 0x01010101u;
                        if (nc >= 0) xw[s] = __vminu4(ld_word(a.u.cat, nc, a.u.ld, quad), static_cast<uint32_t>(K - 1) * 0x01010101u);
                    }
                }
            }
            uint32_t out = 0;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                if (!live || 4 * static_cast<int64_t>(quad) + c >= a.u.n_chains) break;
                const int sh = 8 * c;
                float th[KT], sm[KT];
#pragma unroll
                for (int k = 0; k < KT; ++k) th[k] = sm[k] = 0.0f;
#pragma unroll
                for (int s = 0; s < CAT_SLOTS; ++s) {
                    if (s >= cnt) break;  // uniform over the warp
                    const bool opens = (opens_mask >> s) & 1u, closes = (closes_mask >> s) & 1u;
                    // +-1.0f: w * sign + th in one fused multiply-add rounds exactly as th + (+-w) does
                    const float sign = __uint_as_float(0x3f800000u | (((sg[s] >> sh) & 1u) << 31));
                    const float4* row = reinterpret_cast<const float4*>(mine + s * K * KP + ((xw[s] >> sh) & 0xffu) * KP);
                    float w[4 * NV];
#pragma unroll
                    for (int v = 0; v < NV; ++v) {
                        const float4 q = row[v];
                        w[4 * v] = q.x; w[4 * v + 1] = q.y; w[4 * v + 2] = q.z; w[4 * v + 3] = q.w;
                    }
                    if (opens && closes) {  // a table with one active slot: its sum is the weight itself
#pragma unroll
                        for (int k = 0; k < KT; ++k) th[k] = __fmaf_rn(w[k], sign, th[k]);
                    } else {  // the branches are uniform over the warp and taken outside the category loops
                        if (opens) {  // 0 + t = t (a sum that starts at -0 instead of +0 gives the same logits: th is never -0)
#pragma unroll
                            for (int k = 0; k < KT; ++k) sm[k] = __fmul_rn(w[k], sign);
                        } else {
#pragma unroll
                            for (int k = 0; k < KT; ++k) sm[k] = __fmaf_rn(w[k], sign, sm[k]);
                        }
                        if (closes) {
#pragma unroll
                            for (int k = 0; k < KT; ++k) th[k] = __fadd_rn(th[k], sm[k]);
                        }
                    }
                }
                float best = 0.f, second = -3.0e38f, lmin = 1.0f;
                uint32_t lead = 0;
                U4 r{0, 0, 0, 0};
#pragma unroll
                for (int k = 0; k < KT; ++k) {
                    if (k >= K) break;
                    if ((k & 3) == 0)
                        r = philox4x32_10_rk(static_cast<uint32_t>(node), 4u * (a.u.chain_word0 + static_cast<uint32_t>(quad)) + c, static_cast<uint32_t>(k >> 2), TAG_CAT, a.rk);
                    const uint32_t word = (k & 3) == 0 ? r.x : ((k & 3) == 1 ? r.y : ((k & 3) == 2 ? r.z : r.w));
                    const float u = __uint_as_float(0x3f800000u | (word >> 9)) - 0.99999994039535522461f;  // the 23-bit uniform of u23_open
                    const float l1 = lg2_normal(u) * -0.6931471805599453f;               // -ln u > 0
                    const float p = fmaf(lg2_normal(l1), -0.6931471805599453f, th[k]);   // th - ln(l1)
                    if (k == 0) {
                        best = p;
                        lmin = l1;
                    } else {
                        lmin = fminf(lmin, l1);
                        second = fmaxf(second, fminf(best, p));
                        if (p > best) { best = p; lead = k; }
                    }
                }
                // k_cat_fast's bound: a leader closer to the runner-up than the screen's error is recomputed exactly
                if (!(best - second > MARGIN + 6.0e-7f * rcp_normal(lmin))) lead = cat_exact_argmax(a.u, node, quad, c);
                out |= lead << sh;
            }
            if (live) *reinterpret_cast<uint32_t*>(drow + 4 * static_cast<int64_t>(quad)) = out;
        }
    }
}

// Categorical blocks with 9 to 32 active slots per node (K <= 16, 128 chains or more): k_cat_warp's arithmetic without its
// per-slot registers.  Per pass a lane packs, for each slot, the neighbour's category and the sign of the spin tails of its
// four chains into one word kept in shared memory ([slot][lane]: conflict-free); per-slot facts that are the same for
// every lane (weight row, flags) sit beside it.  STAGE: the node's weight rows are staged in dynamic shared memory as in
// k_cat_warp (pair slots transposed, `slots` rows of K x KP floats per warp); otherwise they are read through L1, a
// column of K values per slot and chain (the lanes of a warp then ask for up to K different addresses per load, which
// is what the staging avoids).
constexpr int CAT_MANY_SLOTS = 32;
struct CatManyArgs {
    CatWarpArgs w;
    int32_t slots;  // STAGE: weight rows staged per warp = the block's largest active slot count
};
template <int KT, bool STAGE>
__global__ void __launch_bounds__(256, 2) k_cat_many(const __grid_constant__ CatManyArgs args) {
    extern __shared__ float4 s_stage4[];  // STAGE: [warps][slots][K][KP]
    __shared__ uint32_t s_slot[8][CAT_MANY_SLOTS][32];
    __shared__ const float* s_wp[8][CAT_MANY_SLOTS];
    __shared__ uint32_t s_flag[8][CAT_MANY_SLOTS];  // bit 0 categorical tail, bit 1 opens a table, bit 2 closes one
    constexpr float MARGIN = 1.2e-5f;
    constexpr int NV = (KT + 3) / 4;
    const CatWarpArgs& a = args.w;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int K = a.u.K;
    const int KP = (K + 3) & ~3;
    float* mine = reinterpret_cast<float*>(s_stage4) + static_cast<size_t>(warp) * args.slots * K * KP;
    for (int node = blockIdx.x * warps + warp; node < a.u.n; node += gridDim.x * warps) {
        const int cnt = __ldg(a.cnt + node);
        const uint32_t first = __ldg(a.first + node);
        int32_t nb0 = -1, nb1 = -1, nb2 = -1, nbc = -1;
        __syncwarp();  // the previous node's reads of the per-slot facts and of the staged weights are done
        if (lane < cnt) {
            const int32_t code = __ldg(a.ent + static_cast<int64_t>(node) * CAT_MANY_SLOTS + lane);
            const DevTable& T = a.u.tabs[code >> 24];
            const int64_t flat = static_cast<int64_t>(node) * T.k + (code & 0xffffff);
            if (T.n_spin > 0) nb0 = __ldg(T.idx[0] + flat);
            if (T.n_spin > 1) nb1 = __ldg(T.idx[1] + flat);
            if (T.n_spin > 2) nb2 = __ldg(T.idx[2] + flat);
            if (T.n_tails > T.n_spin) nbc = __ldg(T.idx[T.n_spin] + flat);
            s_wp[warp][lane] = T.w + flat * T.wdim;
            const bool closes = lane + 1 >= cnt || ((first >> (lane + 1)) & 1u);
            s_flag[warp][lane] = (nbc >= 0 ? 1u : 0u) | (((first >> lane) & 1u) << 1) | (closes ? 4u : 0u);
        }
        __syncwarp();
        if (STAGE) {
            for (int s = 0; s < cnt; ++s) {
                const float* src = s_wp[warp][s];
                float* dst = mine + s * K * KP;
                if (s_flag[warp][s] & 1u) {
                    for (int i = lane; i < K * K; i += 32) {
                        const int own = i / K, x = i - own * K;
                        dst[x * KP + own] = __ldg(src + i);
                    }
                } else {
                    for (int i = lane; i < K; i += 32) dst[i] = __ldg(src + i);
                }
            }
            __syncwarp();
        }
        uint8_t* drow = a.u.dst + static_cast<int64_t>(node) * a.u.ld;
        for (int base = 0; base < a.n_chunks4; base += 32) {  // every lane runs every pass: the entry broadcasts are warp-wide
            const int quad = base + lane;
            const bool live = quad < a.n_chunks4;
            for (int s = 0; s < cnt; ++s) {  // uniform over the warp
                const int32_t n0 = __shfl_sync(0xffffffffu, nb0, s), n1 = __shfl_sync(0xffffffffu, nb1, s), n2 = __shfl_sync(0xffffffffu, nb2, s);
                const int32_t nc = __shfl_sync(0xffffffffu, nbc, s);
                uint32_t v = 0;
                if (live) {
                    uint32_t neg = 0;
                    if (n0 >= 0) neg ^= ~ld_word(a.u.spin, n0, a.u.ld, quad);
                    if (n1 >= 0) neg ^= ~ld_word(a.u.spin, n1, a.u.ld, quad);
                    if (n2 >= 0) neg ^= ~ld_word(a.u.spin, n2, a.u.ld, quad);
                    if (nc >= 0) v = __vminu4(ld_word(a.u.cat, nc, a.u.ld, quad), static_cast<uint32_t>(K - 1) * 0x01010101u);
                    v |= (neg & 0x01010101u) << 7;  // a category is below 16: bit 7 of the byte is free for the sign
                }
                s_slot[warp][s][lane] = v;  // read back by this lane only
            }
            uint32_t out = 0;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                if (!live || 4 * static_cast<int64_t>(quad) + c >= a.u.n_chains) break;
                const int sh = 8 * c;
                float th[KT], sm[KT];
#pragma unroll
                for (int k = 0; k < KT; ++k) th[k] = sm[k] = 0.0f;
                for (int s = 0; s < cnt; ++s) {
                    const uint32_t b = (s_slot[warp][s][lane] >> sh) & 0xffu;
                    const uint32_t flag = s_flag[warp][s];
                    const float sign = __uint_as_float(0x3f800000u | ((b >> 7) << 31));  // +-1.0f: w * sign + th rounds exactly as th + (+-w)
                    float w[4 * NV];
                    if (STAGE) {
                        const float4* row = reinterpret_cast<const float4*>(mine + s * K * KP + (b & 0x7fu) * KP);  // an untailed slot has category 0
#pragma unroll
                        for (int v = 0; v < NV; ++v) {
                            const float4 q = row[v];
                            w[4 * v] = q.x; w[4 * v + 1] = q.y; w[4 * v + 2] = q.z; w[4 * v + 3] = q.w;
                        }
                    } else {
                        const float* col = s_wp[warp][s] + ((flag & 1u) ? (b & 0x7fu) : 0u);
                        const int stride = (flag & 1u) ? K : 1;
#pragma unroll
                        for (int k = 0; k < KT; ++k) w[k] = k < K ? __ldg(col + k * stride) : 0.0f;
                    }
                    if ((flag & 6u) == 6u) {  // a table with one active slot: its sum is the weight itself
#pragma unroll
                        for (int k = 0; k < KT; ++k) th[k] = __fmaf_rn(w[k], sign, th[k]);
                    } else {  // the branches are uniform over the warp and taken outside the category loops
                        if (flag & 2u) {  // 0 + t = t (a sum that starts at -0 instead of +0 gives the same logits: th is never -0)
#pragma unroll
                            for (int k = 0; k < KT; ++k) sm[k] = __fmul_rn(w[k], sign);
                        } else {
#pragma unroll
                            for (int k = 0; k < KT; ++k) sm[k] = __fmaf_rn(w[k], sign, sm[k]);
                        }
                        if (flag & 4u) {
#pragma unroll
                            for (int k = 0; k < KT; ++k) th[k] = __fadd_rn(th[k], sm[k]);
                        }
                    }
                }
                float best = 0.f, second = -3.0e38f, lmin = 1.0f;
                uint32_t lead = 0;
                U4 r{0, 0, 0, 0};
#pragma unroll
                for (int k = 0; k < KT; ++k) {
                    if (k >= K) break;
                    if ((k & 3) == 0)
                        r = philox4x32_10_rk(static_cast<uint32_t>(node), 4u * (a.u.chain_word0 + static_cast<uint32_t>(quad)) + c, static_cast<uint32_t>(k >> 2), TAG_CAT, a.rk);
                    const uint32_t word = (k & 3) == 0 ? r.x : ((k & 3) == 1 ? r.y : ((k & 3) == 2 ? r.z : r.w));
                    const float u = __uint_as_float(0x3f800000u | (word >> 9)) - 0.99999994039535522461f;  // the 23-bit uniform of u23_open
                    const float l1 = lg2_normal(u) * -0.6931471805599453f;
                    const float p = fmaf(lg2_normal(l1), -0.6931471805599453f, th[k]);
                    if (k == 0) {
                        best = p;
                        lmin = l1;
                    } else {
                        lmin = fminf(lmin, l1);
                        second = fmaxf(second, fminf(best, p));
                        if (p > best) { best = p; lead = k; }
                    }
                }
                if (!(best - second > MARGIN + 6.0e-7f * rcp_normal(lmin))) lead = cat_exact_argmax(a.u, node, quad, c);
                out |= lead << sh;
            }
            if (live) *reinterpret_cast<uint32_t*>(drow + 4 * static_cast<int64_t>(quad)) = out;
        }
    }
}

// Threshold tables for spin blocks whose nodes see at most 8 neighbour spins through single-spin-tail tables:
// lut[node][cfg] = the largest 32-bit random word for which the node becomes 1 when its neighbours are cfg
// (bit j = state of the j-th active neighbour slot in table order).  gamma is accumulated exactly as in
// k_spin_generic, and u <= p  <=>  (r >> 8) <= floor(p * 2^24)  <=>  r <= (floor(p * 2^24) << 8 | 0xff).
// `nodes` (nullable): the block's nodes that get a table, in table order; null = every node, in node order.
__global__ void __launch_bounds__(256) k_build_lut(const DevTable* tabs, int32_t n_tabs, int32_t n, uint32_t* lut, const int32_t* nodes) {
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint32_t cfg = static_cast<uint32_t>(gid) & (LUT_SIZE - 1);
    if ((gid >> LUT_BITS) >= n) return;
    const int64_t node = nodes ? nodes[gid >> LUT_BITS] : (gid >> LUT_BITS);
    float gamma = 0.f;
    int bit = 0;
    for (int t = 0; t < n_tabs; ++t) {
        const DevTable T = tabs[t];
        float gs = 0.f;
        for (int j = 0; j < T.k; ++j) {
            const int64_t flat = node * T.k + j;
            if (!T.active[flat]) continue;
            float sp = 1.0f;
            if (T.n_spin == 1) {
                sp = ((cfg >> bit) & 1u) ? 1.0f : -1.0f;
                ++bit;
            }
            gs = __fadd_rn(gs, __fmul_rn(T.w[flat], sp));
        }
        gamma = __fadd_rn(gamma, gs);
    }
    const float p = det_sigmoid(__fmul_rn(gamma, 2.0f));
    const uint32_t fl = static_cast<uint32_t>(__fmul_rn(p, 16777216.0f));  // exact: p*2^24 <= 2^24
    lut[gid] = fl >= 16777216u ? 0xffffffffu : ((fl << 8) | 0xffu);
}

struct LutArgs {
    const int32_t* nbr;    // [n][8] global spin positions, -1 = unused slot
    const uint32_t* lut;   // [n][256]
    const uint8_t* spin;
    uint8_t* dst;
    int64_t ld;
    int32_t n;
    int32_t n_chunks;      // ld / 16
    uint32_t chain_word0;
    PhiloxRoundKeys rk;    // round keys of the block key
    // fused moment observer (ACC only): row of <s_i> per node, row of <s_i s_j> per (node, slot), -1 = not owned here
    int64_t n_chains;
    const int32_t* m1_row;
    const int32_t* m2_row;
    long long* sums;
};

// Bytes 0xff for the chains of word q of chunk ch that exist (chain index < n_chains).
__device__ __forceinline__ uint32_t valid_mask(int64_t n_chains, int ch, int q) {
    const int64_t left = n_chains - (16 * static_cast<int64_t>(ch) + 4 * q);
    if (left >= 4) return 0xffffffffu;
    if (left <= 0) return 0u;
    return 0xffffffffu >> (8 * (4 - static_cast<int>(left)));
}
__device__ __forceinline__ uint32_t maj3(uint32_t a, uint32_t b, uint32_t c) { return (a & b) | (c & (a | b)); }

// Bit-sliced counters: plane[p] holds bit p of 32 independent counts, one per bit position of a state word
// (bit j of byte b = "neighbour slot j differs from the new spin" for the chain in byte b).  Adding the four words of a
// pass costs 17 logic ops for all 8 slots and 4 chains at once; counts up to 63 fit, i.e. 15 passes of 4 words.
struct SliceCounter {
    uint32_t p0 = 0, p1 = 0, p2 = 0, p3 = 0, p4 = 0, p5 = 0;
    __device__ __forceinline__ void add4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
        const uint32_t s1 = a ^ b ^ c, c1 = maj3(a, b, c);  // a+b+c = s1 + 2 c1
        const uint32_t ones = s1 ^ d, c2 = s1 & d;           // + d
        const uint32_t twos = c1 ^ c2, fours = c1 & c2;
        uint32_t k = p0 & ones;
        p0 ^= ones;
        uint32_t k2 = maj3(p1, twos, k);
        p1 ^= twos ^ k;
        k = maj3(p2, fours, k2);
        p2 ^= fours ^ k2;
        k2 = p3 & k;
        p3 ^= k;
        k = p4 & k2;
        p4 ^= k2;
        p5 ^= k;
    }
    // count of bit position `j` summed over the four bytes of the word
    __device__ __forceinline__ uint32_t total(int j) const {
        const uint32_t m = 0x01010101u << j;
        return __popc(p0 & m) + 2 * __popc(p1 & m) + 4 * __popc(p2 & m) + 8 * __popc(p3 & m) + 16 * __popc(p4 & m) + 32 * __popc(p5 & m);
    }
};
constexpr int ACC_SEGMENT_PASSES = 15;  // 15 passes x 4 words = 60 <= 63

// Threshold-table spin update: one warp per node, each lane 16 chains per pass.  The neighbour configuration of four
// chains is assembled with shifts inside one 32-bit word (state bytes are 0/1), then one shared-memory lookup and one
// compare per chain replace the field accumulation and the sigmoid.
// ACC: the moment observer fused into the update (moment.rs:205-233 for first moments and pair products): the warp
// that updates node i is the only one that touches i's rows, so the sums are updated without atomics.  A pair row is
// owned by the endpoint updated later in the sweep, when both values are final.  Disagreements with each neighbour
// slot are counted in bit-sliced counters and reduced once per node.
// COHERENT: neighbour rows may have been written earlier in the same launch (persistent multi-sweep kernel), so they are
// read through L2 (ld.global.cg) instead of the read-only path.
// One node of the threshold-table update by one warp.  `row` selects the node's neighbour list and table (equal to
// `node` unless the block keeps tables only for some of its nodes), `m2_at` the first of its pair-row entries.
template <bool ACC, bool COHERENT>
__device__ __forceinline__ void lut_node_update(const LutArgs& a, uint32_t* my, int node, int64_t row, int64_t m2_at) {
    const int lane = threadIdx.x & 31;
    const uint4* src = reinterpret_cast<const uint4*>(a.lut + row * LUT_SIZE);
    __syncwarp();
    reinterpret_cast<uint4*>(my)[lane] = __ldg(src + lane);
    reinterpret_cast<uint4*>(my)[lane + 32] = __ldg(src + lane + 32);
    int32_t nb = lane < LUT_BITS ? __ldg(a.nbr + row * LUT_BITS + lane) : -1;
    int32_t my_row = -1;
    uint32_t own = 0;
    if (ACC) {
        if (lane < LUT_BITS) my_row = __ldg(a.m2_row + m2_at + lane);
        else if (lane == LUT_BITS) my_row = __ldg(a.m1_row + node);
        own = __ballot_sync(0xffffffffu, my_row >= 0);
    }
    __syncwarp();
    int32_t nbj[LUT_BITS];
#pragma unroll
    for (int j = 0; j < LUT_BITS; ++j) nbj[j] = __shfl_sync(0xffffffffu, nb, j);
    uint8_t* drow = a.dst + static_cast<int64_t>(node) * a.ld;
    uint32_t mine = 0;  // lane j < 8: disagreements with slot j; lane 8: number of ones
    for (int seg = 0; seg < a.n_chunks; seg += 32 * ACC_SEGMENT_PASSES) {
        const int seg_end = min(a.n_chunks, seg + 32 * ACC_SEGMENT_PASSES);
        SliceCounter cnt;
        uint32_t ones = 0;
        for (int ch = seg + lane; ch < seg_end; ch += 32) {
            uint4 v[LUT_BITS];
#pragma unroll
            for (int j = 0; j < LUT_BITS; ++j) {
                v[j] = make_uint4(0, 0, 0, 0);
                if (nbj[j] >= 0) {
                    const uint4* src_row = reinterpret_cast<const uint4*>(a.spin + static_cast<int64_t>(nbj[j]) * a.ld) + ch;
                    v[j] = COHERENT ? __ldcg(src_row) : __ldg(src_row);
                }
            }
            uint32_t cfg[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < LUT_BITS; ++j) {
                cfg[0] += v[j].x << j;
                cfg[1] += v[j].y << j;
                cfg[2] += v[j].z << j;
                cfg[3] += v[j].w << j;
            }
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const U4 r = philox4x32_10_rk(static_cast<uint32_t>(node), a.chain_word0 + 4u * ch + q, 0u, TAG_SPIN, a.rk);
                uint32_t w = 0;
                w |= (r.x <= my[cfg[q] & 0xffu]) ? 1u : 0u;
                w |= (r.y <= my[(cfg[q] >> 8) & 0xffu]) ? 0x100u : 0u;
                w |= (r.z <= my[(cfg[q] >> 16) & 0xffu]) ? 0x10000u : 0u;
                w |= (r.w <= my[cfg[q] >> 24]) ? 0x1000000u : 0u;
                o[q] = w;
            }
            reinterpret_cast<uint4*>(drow)[ch] = make_uint4(o[0], o[1], o[2], o[3]);
            if (ACC && own) {
                uint32_t d[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) d[q] = cfg[q] ^ (o[q] * 255u);  // bit j of a byte: neighbour j differs from the new spin
                if (16 * static_cast<int64_t>(ch + 1) > a.n_chains) {        // ragged last chunk: drop chains that do not exist
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t vm = valid_mask(a.n_chains, ch, q);
                        d[q] &= vm;
                        o[q] &= vm;
                    }
                }
                cnt.add4(d[0], d[1], d[2], d[3]);
                ones += __popc(o[0] + (o[1] << 1) + (o[2] << 2) + (o[3] << 3));
            }
        }
        if (ACC && own) {
            ones = __reduce_add_sync(0xffffffffu, ones);
            if (lane == LUT_BITS) mine += ones;
#pragma unroll
            for (int j = 0; j < LUT_BITS; ++j)
                if ((own >> j) & 1u) {
                    const uint32_t t = __reduce_add_sync(0xffffffffu, cnt.total(j));
                    if (lane == j) mine += t;
                }
        }
    }
    if (ACC && my_row >= 0) {
        const long long val = lane == LUT_BITS ? 2ll * mine - a.n_chains : a.n_chains - 2ll * mine;
        if (COHERENT) __stcg(a.sums + my_row, __ldcg(a.sums + my_row) + val);
        else a.sums[my_row] += val;
    }
}
template <bool ACC, bool COHERENT>
__device__ __forceinline__ void lut_block_update(const LutArgs& a, uint32_t* my) {
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int node = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; node < a.n; node += warps)
        lut_node_update<ACC, COHERENT>(a, my, node, node, static_cast<int64_t>(node) * LUT_BITS);
}

template <bool ACC>
__global__ void __launch_bounds__(256, 4) k_spin_lut(const __grid_constant__ LutArgs a) {
    __shared__ uint32_t s_lut[8][LUT_SIZE];
    lut_block_update<ACC, false>(a, s_lut[threadIdx.x >> 5]);
}

// Few chains (at most 256, i.e. at most 16 chunks of 16): a warp per node would leave most lanes idle and stage a whole
// 1 KiB table for a handful of lookups.  Here one THREAD updates one node for one chunk of 16 chains: the neighbour
// list and the table entries it needs come through the read-only cache, threads of a warp work on different nodes.
// Same bits as k_spin_lut (same configuration byte, same table, same noise).  ACC adds each thread's share of the
// node's <s_i> row and of the pair rows the node owns with atomics (several threads may share a node).
template <bool ACC>
__global__ void __launch_bounds__(256) k_spin_lut_thread(const __grid_constant__ LutArgs a) {
    const int64_t total = static_cast<int64_t>(a.n) * a.n_chunks;
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int node = static_cast<int>(t / a.n_chunks), ch = static_cast<int>(t % a.n_chunks);
        const int4 n0 = __ldg(reinterpret_cast<const int4*>(a.nbr + static_cast<int64_t>(node) * LUT_BITS));
        const int4 n1 = __ldg(reinterpret_cast<const int4*>(a.nbr + static_cast<int64_t>(node) * LUT_BITS) + 1);
        const int32_t nb[LUT_BITS] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
        uint32_t cfg[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < LUT_BITS; ++j)
            if (nb[j] >= 0) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(a.spin + static_cast<int64_t>(nb[j]) * a.ld) + ch);
                cfg[0] += v.x << j;
                cfg[1] += v.y << j;
                cfg[2] += v.z << j;
                cfg[3] += v.w << j;
            }
        const uint32_t* L = a.lut + static_cast<int64_t>(node) * LUT_SIZE;
        uint32_t o[4] = {0, 0, 0, 0};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (16ll * ch + 4 * q >= a.n_chains) continue;  // nothing but padding in this word
            const U4 r = philox4x32_10_rk(static_cast<uint32_t>(node), a.chain_word0 + 4u * ch + q, 0u, TAG_SPIN, a.rk);
            uint32_t w = 0;
            w |= (r.x <= __ldg(L + (cfg[q] & 0xffu))) ? 1u : 0u;
            w |= (r.y <= __ldg(L + ((cfg[q] >> 8) & 0xffu))) ? 0x100u : 0u;
            w |= (r.z <= __ldg(L + ((cfg[q] >> 16) & 0xffu))) ? 0x10000u : 0u;
            w |= (r.w <= __ldg(L + (cfg[q] >> 24))) ? 0x1000000u : 0u;
            o[q] = w;
        }
        reinterpret_cast<uint4*>(a.dst + static_cast<int64_t>(node) * a.ld)[ch] = make_uint4(o[0], o[1], o[2], o[3]);
        if (ACC) {
            uint32_t vm[4];
            int valid = 0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                vm[q] = valid_mask(a.n_chains, ch, q) & 0x01010101u;
                valid += __popc(vm[q]);
            }
            const int32_t row1 = __ldg(a.m1_row + node);
            if (row1 >= 0) {
                const int ones = __popc(o[0] & vm[0]) + __popc(o[1] & vm[1]) + __popc(o[2] & vm[2]) + __popc(o[3] & vm[3]);
                atomicAdd(reinterpret_cast<unsigned long long*>(a.sums) + row1, static_cast<unsigned long long>(static_cast<long long>(2 * ones - valid)));
            }
            const int4 r0 = __ldg(reinterpret_cast<const int4*>(a.m2_row + static_cast<int64_t>(node) * LUT_BITS));
            const int4 r1 = __ldg(reinterpret_cast<const int4*>(a.m2_row + static_cast<int64_t>(node) * LUT_BITS) + 1);
            const int32_t rows[LUT_BITS] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
            for (int j = 0; j < LUT_BITS; ++j)
                if (rows[j] >= 0) {
                    int dis = 0;  // chains in which neighbour j differs from the new spin
#pragma unroll
                    for (int q = 0; q < 4; ++q) dis += __popc(((cfg[q] >> j) ^ o[q]) & vm[q]);
                    atomicAdd(reinterpret_cast<unsigned long long*>(a.sums) + rows[j], static_cast<unsigned long long>(static_cast<long long>(valid - 2 * dis)));
                }
        }
    }
}

// Persistent multi-sweep variant for cache-resident programs: one cooperative launch walks a list of block updates
// (sweep-major, blocks in sampling order) with a grid-wide barrier after each, instead of one launch per block update.
// For small models a block update takes a microsecond or two and the launches themselves dominate.
__global__ void __launch_bounds__(256, 2) k_spin_lut_persistent(const LutArgs* steps, const uint8_t* acc, int32_t n_steps) {
    __shared__ uint32_t s_lut[8][LUT_SIZE];
    cooperative_groups::grid_group grid = cooperative_groups::this_grid();
    for (int32_t i = 0; i < n_steps; ++i) {
        const LutArgs a = steps[i];  // by value: the round keys stay in registers across the update's stores
        if (__ldg(acc + i)) lut_block_update<true, true>(a, s_lut[threadIdx.x >> 5]);
        else lut_block_update<false, true>(a, s_lut[threadIdx.x >> 5]);
        grid.sync();
    }
}

// Sequential-sum spin update for blocks whose nodes have more single-spin-tail neighbour slots than a threshold table
// covers (entry lists in rows of SEQ_MAX, bias entries included; any length).  Same data movement as k_spin_lut — one warp per
// node, 16 chains per lane per pass, one 16-byte load per neighbour row — but the field is accumulated entry by
// entry in the canonical order (per table from zero, tables left to right), exactly as k_spin_generic does, so the
// states are the same bits.  The sigmoid is approximated first (2^x and reciprocal units); only a draw within 4e-6 of
// it (four times the approximation's worst error) is redone with the deterministic sigmoid.
constexpr int SEQ_MAX = 32;
// Entry lists from the slot tables: per node the active slots in table order, slot order, in rows of SEQ_MAX entries;
// nbr = -1 for an entry without a tail (a bias); bit e of first[row] marks the first entry of a table; cnt[row] = entries
// in the row.  Row `node` holds a node's first SEQ_MAX entries; a node with more continues in rows overflow[node],
// overflow[node] + 1, ... (rows n and up; overflow[node] = -1 for the others).
__global__ void __launch_bounds__(256) k_build_seq(const DevTable* tabs, int32_t n_tabs, int32_t n, const int32_t* overflow, int32_t* ent_nbr, float* ent_w,
                                                   uint32_t* ent_first, int32_t* ent_cnt) {
    const int64_t node = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (node >= n) return;
    int e = 0;          // entry inside the current row
    int64_t row = node;
    int64_t next = overflow[node];
    uint32_t first = 0;
    for (int t = 0; t < n_tabs; ++t) {
        const DevTable T = tabs[t];
        bool started = false;
        for (int j = 0; j < T.k; ++j) {
            const int64_t flat = node * T.k + j;
            if (!T.active[flat]) continue;
            if (e == SEQ_MAX) {  // row full: close it and continue in the node's next overflow row
                ent_first[row] = first;
                ent_cnt[row] = SEQ_MAX;
                row = next++;
                e = 0;
                first = 0;
            }
            if (!started) first |= 1u << e;
            started = true;
            ent_nbr[row * SEQ_MAX + e] = T.n_spin == 1 ? T.idx[0][flat] : -1;
            ent_w[row * SEQ_MAX + e] = T.w[flat];
            ++e;
        }
    }
    ent_first[row] = first;
    ent_cnt[row] = e;
    for (; e < SEQ_MAX; ++e) {
        ent_nbr[row * SEQ_MAX + e] = -1;
        ent_w[row * SEQ_MAX + e] = 0.0f;
    }
}
struct SeqArgs {
    const int32_t* nbr;     // [rows][SEQ_MAX], rows = n + overflow rows
    const float* w;         // [rows][SEQ_MAX]
    const uint32_t* first;  // [rows]
    const int32_t* cnt;     // [rows]
    const int32_t* overflow;  // [n] first overflow row of a node with more than SEQ_MAX entries, -1 otherwise
    const int32_t* n_rows;    // [n] rows of the node (1 unless it overflows)
    const uint8_t* spin;
    uint8_t* dst;
    int64_t ld;
    int32_t n;
    int32_t n_chunks;       // ld / 16
    uint32_t chain_word0;
    PhiloxRoundKeys rk;
    // fused moment observer (ACC only): row of <s_i> per node, row of <s_i s_j> per (node, entry), -1 = not owned here
    int64_t n_chains;
    const int32_t* m1_row;
    const int32_t* m2_row;
    long long* sums;
    // Work distribution: warps take nodes from a shared counter (zeroed before the launch), in the order of `order`
    // (most entries first).  Node costs differ by the entry count, so a fixed assignment leaves a long tail.
    const int32_t* order;   // [n] permutation of the block's nodes
    int32_t* counter;
    // Split field tables (nullptr = none): split_row[node] >= 0 is the node's row in split_tab / split_margin.
    const int32_t* split_row;
    const float* split_tab;     // [rows][2][256]
    const float* split_margin;  // [rows]
};
// Next node for this warp, or -1 when the block is done.
__device__ __forceinline__ int take_node(const SeqArgs& a) {
    int i = 0;
    if ((threadIdx.x & 31) == 0) i = atomicAdd(a.counter, 1);
    i = __shfl_sync(0xffffffffu, i, 0);
    return i < a.n ? __ldg(a.order + i) : -1;
}
// The exact draw rule u <= sigmoid(2 gamma) (spin_gibbs.rs:95-97), out of line: k_spin_seq needs it for about one draw in 10^5.
__device__ __noinline__ bool exact_spin_draw(float gamma, uint32_t r) { return u24(r) <= det_sigmoid(__fmul_rn(gamma, 2.0f)); }

// ACC: the moment observer fused in, as in k_spin_lut<true>: this node's <s_i> row and the pair rows it owns (it is the
// endpoint updated later in the sweep) are accumulated without atomics.  The new spin is known only after the last
// entry, so the owned neighbours' rows are read a second time (they were loaded moments before: cache hits) and
// compared with the new bytes.
// Four CTAs per SM (64 registers, a few spilled words): measured faster than three without spills, and than 8 chains per lane.
template <bool ACC>
__device__ __forceinline__ void seq_node_update(const SeqArgs& a, int node) {
    const int lane = threadIdx.x & 31;
    int32_t nb = __ldg(a.nbr + static_cast<int64_t>(node) * SEQ_MAX + lane);
    float wv = __ldg(a.w + static_cast<int64_t>(node) * SEQ_MAX + lane);
    uint32_t first = __ldg(a.first + node);
    int cnt = __ldg(a.cnt + node);
    const int n_rows = __ldg(a.n_rows + node);       // more than one only for a node with more than SEQ_MAX entries
    const int64_t overflow = __ldg(a.overflow + node);
    uint8_t* drow = a.dst + static_cast<int64_t>(node) * a.ld;
    int32_t my_row = -1, row1 = -1;
    uint32_t own = 0;        // entries whose pair row this node owns
    uint32_t mine = 0;       // lane e: disagreements with the neighbour of entry e
    uint32_t ones_total = 0; // lane 0: chains in which the new spin is 1
    if (ACC) {
        my_row = __ldg(a.m2_row + static_cast<int64_t>(node) * SEQ_MAX + lane);
        row1 = __ldg(a.m1_row + node);
        own = __ballot_sync(0xffffffffu, my_row >= 0);
    }
    for (int base = 0; base < a.n_chunks; base += 32) {  // every lane runs every pass: the entry broadcasts are warp-wide
        const int ch = base + lane;
        const bool live = ch < a.n_chunks;
        float gam[16], part[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) gam[i] = part[i] = 0.0f;
        // four neighbour rows are always in flight: the row of entry e + 4 is requested when entry e is consumed
        const uint4 ones = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);  // no tail: the product over tails is +1
        auto row_of = [&](int e) {
            const int32_t nbe = __shfl_sync(0xffffffffu, nb, e);
            return nbe >= 0 && live ? __ldg(reinterpret_cast<const uint4*>(a.spin + static_cast<int64_t>(nbe) * a.ld) + ch) : ones;
        };
        for (int seg = 0; seg < n_rows; ++seg) {
            if (n_rows > 1) {  // a long entry list: its rows are (re)loaded pass by pass
                const int64_t row = seg == 0 ? node : overflow + seg - 1;
                nb = __ldg(a.nbr + row * SEQ_MAX + lane);
                wv = __ldg(a.w + row * SEQ_MAX + lane);
                first = __ldg(a.first + row);
                cnt = __ldg(a.cnt + row);
            }
            uint4 ring[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) ring[k] = k < cnt ? row_of(k) : ones;
            for (int e0 = 0; e0 < cnt; e0 += 4) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int e = e0 + k;
                    if (e >= cnt) break;  // uniform over the warp
                    const uint4 v = ring[k];
                    if (e + 4 < cnt) ring[k] = row_of(e + 4);
                    const float we = __shfl_sync(0xffffffffu, wv, e);
                    if ((first >> e) & 1u) {  // a new table: close the previous one
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            gam[i] = __fadd_rn(gam[i], part[i]);
                            part[i] = 0.0f;
                        }
                    }
                    // 2 s - 1 as a float per chain with one byte permute: the bytes of t are 0x3f (spin +1) or 0xbf (spin -1),
                    // the top byte of +-1.0f; the other three bytes (0x80, 0, 0) come from the constant.  Then one fused
                    // multiply-add: w * (+-1) is exact, so the sum rounds as the reference's add does.  (The integer pipe is
                    // the busy one: this is one of its operations per neighbour and chain instead of two.)
                    const uint32_t t[4] = {((v.x ^ 0x01010101u) << 7) | 0x3f3f3f3fu, ((v.y ^ 0x01010101u) << 7) | 0x3f3f3f3fu,
                                           ((v.z ^ 0x01010101u) << 7) | 0x3f3f3f3fu, ((v.w ^ 0x01010101u) << 7) | 0x3f3f3f3fu};
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const float sp = __uint_as_float(__byte_perm(t[q], 0x00800000u, 0x0654u | (c << 12)));
                            part[4 * q + c] = __fmaf_rn(sp, we, part[4 * q + c]);
                        }
                }
            }
        }
        // d = 2^24 (u - p) with the approximate sigmoid; the spin is the sign of d.  One test per pass finds the draws that
        // are too close to call (within 4e-6 of p): only then the exact rule runs, for those draws.
        uint32_t o[4];
        float nearest = 16777216.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const U4 r = philox4x32_10_rk(static_cast<uint32_t>(node), a.chain_word0 + 4u * ch + q, 0u, TAG_SPIN, a.rk);
            const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
            o[q] = 0;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float gamma = __fadd_rn(gam[4 * q + c], part[4 * q + c]);
                gam[4 * q + c] = gamma;
                float ex, p24;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(gamma * -2.885390081777927f));
                asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(p24) : "f"(fmaf(ex, 5.9604644775390625e-8f, 5.9604644775390625e-8f)));  // 2^24 p
                const float d = __uint2float_rn(rr[c] >> 8) - p24;
                part[4 * q + c] = d;
                nearest = fminf(nearest, fabsf(d));
                o[q] |= (__float_as_uint(d) >> 31) << (8 * c);
            }
        }
        if (nearest <= 67.2f) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const U4 r = philox4x32_10_rk(static_cast<uint32_t>(node), a.chain_word0 + 4u * ch + q, 0u, TAG_SPIN, a.rk);
                const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (fabsf(part[4 * q + c]) <= 67.2f)
                        o[q] = (o[q] & ~(1u << (8 * c))) | ((exact_spin_draw(gam[4 * q + c], rr[c]) ? 1u : 0u) << (8 * c));
            }
        }
        if (live) reinterpret_cast<uint4*>(drow)[ch] = make_uint4(o[0], o[1], o[2], o[3]);
        if (ACC && (own | static_cast<uint32_t>(row1 >= 0))) {
            uint32_t vm[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) vm[q] = live ? (valid_mask(a.n_chains, ch, q) & 0x01010101u) : 0u;  // chains that exist
            if (row1 >= 0) {
                const uint32_t c = __popc(o[0] & vm[0]) + __popc(o[1] & vm[1]) + __popc(o[2] & vm[2]) + __popc(o[3] & vm[3]);
                const uint32_t t = __reduce_add_sync(0xffffffffu, c);
                if (lane == 0) ones_total += t;
            }
            for (uint32_t left = own; left; left &= left - 1) {  // uniform over the warp
                const int e = __ffs(left) - 1;
                const int32_t nbe = __shfl_sync(0xffffffffu, nb, e);
                uint32_t c = 0;
                if (live) {
                    const uint4 v = __ldg(reinterpret_cast<const uint4*>(a.spin + static_cast<int64_t>(nbe) * a.ld) + ch);
                    c = __popc((v.x ^ o[0]) & vm[0]) + __popc((v.y ^ o[1]) & vm[1]) + __popc((v.z ^ o[2]) & vm[2]) + __popc((v.w ^ o[3]) & vm[3]);
                }
                const uint32_t t = __reduce_add_sync(0xffffffffu, c);
                if (lane == e) mine += t;
            }
        }
    }
    if (ACC) {
        if (my_row >= 0) a.sums[my_row] += a.n_chains - 2ll * mine;
        if (lane == 0 && row1 >= 0) a.sums[row1] += 2ll * ones_total - a.n_chains;
    }
}
// Split field tables for sequential-sum nodes with one entry row (at most 32 neighbour entries): the field is looked
// up as T0[configuration of neighbours 0..7] + T1[neighbours 8..15] (+ T2[16..23] + T3[24..31] for a node with more than
// 16 neighbours) instead of being added entry by entry.  The tables (T0 also carries the entries without a tail) are
// the real partial sums rounded once, so the looked-up field differs from the canonical sequential f32 sum by a few
// rounding errors of the summed |w| at most.  The draw is decided from it only when u is farther from the probability
// than that bound allows (split_margin, in units of 2^-24: the approximate sigmoid's 67.2 plus the field bound pushed
// through the sigmoid's steepest slope); the other draws — a few in 10^5 — take the canonical sum (exact_seq_gamma)
// and the exact rule, so the states are the bits of k_spin_generic.
// split_row[node] = 2 * (first 256-entry table of the node) + (1 if the node has four tables, 0 if two), -1 = none.
constexpr int SPLIT_BITS = 32;
constexpr int SPLIT_TAB = 1024;  // floats a warp stages at most: four tables of 256
constexpr int SPLIT_MIN_CHUNKS = 16;  // states with fewer than 256 chains would read kilobytes of tables per node for a handful of lookups
__global__ void __launch_bounds__(256) k_build_split(const int32_t* split_nodes, const int32_t* split_row, const int32_t* ent_nbr, const float* ent_w,
                                                     const int32_t* ent_cnt, float* tab, float* margin, float extra_margin) {
    const int node = split_nodes[blockIdx.x];
    const int32_t code = split_row[node];
    const int64_t at = static_cast<int64_t>(code >> 1) * 256;
    const int groups = (code & 1) ? 4 : 2;
    const int c = threadIdx.x;  // configuration byte
    const int cnt = ent_cnt[node];
    double S0 = 0.0, S1 = 0.0, S2 = 0.0, S3 = 0.0, mag = 0.0;
    int rank = 0;
    for (int e = 0; e < cnt; ++e) {
        const double w = static_cast<double>(ent_w[static_cast<int64_t>(node) * SEQ_MAX + e]);
        mag += fabs(w);
        if (ent_nbr[static_cast<int64_t>(node) * SEQ_MAX + e] < 0) {
            S0 += w;
        } else {
            const double t = ((c >> (rank & 7)) & 1) ? w : -w;
            if (rank < 8) S0 += t;
            else if (rank < 16) S1 += t;
            else if (rank < 24) S2 += t;
            else S3 += t;
            ++rank;
        }
    }
    tab[at + c] = static_cast<float>(S0);
    tab[at + 256 + c] = static_cast<float>(S1);
    if (groups == 4) {
        tab[at + 512 + c] = static_cast<float>(S2);
        tab[at + 768 + c] = static_cast<float>(S3);
    }
    // |looked-up field - canonical field| <= (2 cnt + 6) 2^-24 sum|w| (one rounding per add of either route, table
    // closings included); times 2 (the sigmoid's argument is twice the field) times 1/4 (its steepest slope) times 2^24,
    // with a tenth on top for the second-order terms.
    if (c == 0) margin[node] = 67.2f + 1.0f + static_cast<float>(0.55 * (2.0 * cnt + 6.0) * mag) + extra_margin;
}
// The canonical field of one node and chain: per table from zero, entries left to right, tables left to right.
__device__ __noinline__ float exact_seq_gamma(const SeqArgs& a, int node, int64_t chain) {
    const int64_t at = static_cast<int64_t>(node) * SEQ_MAX;
    const uint32_t first = __ldg(a.first + node);
    const int cnt = __ldg(a.cnt + node);
    float gam = 0.0f, part = 0.0f;
    for (int e = 0; e < cnt; ++e) {
        if ((first >> e) & 1u) {
            gam = __fadd_rn(gam, part);
            part = 0.0f;
        }
        const int32_t nbe = __ldg(a.nbr + at + e);
        float sp = 1.0f;
        if (nbe >= 0) sp = a.spin[static_cast<int64_t>(nbe) * a.ld + chain] ? 1.0f : -1.0f;
        part = __fmaf_rn(sp, __ldg(a.w + at + e), part);
    }
    return __fadd_rn(gam, part);
}
// d = 2^24 (u - p) from the looked-up field and the approximate sigmoid.
template <int NH>
__device__ __forceinline__ float split_screen(const float* tab, const uint32_t (&cfg)[NH][4], int q, int c, uint32_t r) {
    float gamma = tab[(cfg[0][q] >> (8 * c)) & 0xffu] + tab[256 + ((cfg[1][q] >> (8 * c)) & 0xffu)];
    if (NH == 4) gamma += tab[512 + ((cfg[2][q] >> (8 * c)) & 0xffu)] + tab[768 + ((cfg[3][q] >> (8 * c)) & 0xffu)];
    float ex, p24;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(gamma * -2.885390081777927f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(p24) : "f"(fmaf(ex, 5.9604644775390625e-8f, 5.9604644775390625e-8f)));
    return __uint2float_rn(r >> 8) - p24;
}
template <bool ACC, int NH>
__device__ __forceinline__ void split_node_update(const SeqArgs& a, float* tab, int node, int64_t first_table) {
    const int lane = threadIdx.x & 31;
    const uint4* src = reinterpret_cast<const uint4*>(a.split_tab + first_table * 256);
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 2 * NH; ++k) reinterpret_cast<uint4*>(tab)[lane + 32 * k] = __ldg(src + lane + 32 * k);
    const float margin = __ldg(a.split_margin + node);
    const int32_t nb = __ldg(a.nbr + static_cast<int64_t>(node) * SEQ_MAX + lane);
    const uint32_t tails = __ballot_sync(0xffffffffu, nb >= 0);
    // lane j: the neighbour whose spin is bit j of the configuration (the j-th entry with a tail)
    const uint32_t src_lane = __fns(tails, 0, lane + 1);
    int32_t tnb = __shfl_sync(0xffffffffu, nb, static_cast<int>(src_lane & 31u));
    if (src_lane > 31u) tnb = -1;
    uint8_t* drow = a.dst + static_cast<int64_t>(node) * a.ld;
    int32_t my_row = -1, row1 = -1;
    uint32_t own = 0, mine = 0, ones_total = 0;
    if (ACC) {
        my_row = __ldg(a.m2_row + static_cast<int64_t>(node) * SEQ_MAX + lane);
        row1 = __ldg(a.m1_row + node);
        own = __ballot_sync(0xffffffffu, my_row >= 0);
    }
    __syncwarp();
    for (int seg = 0; seg < a.n_chunks; seg += 32 * ACC_SEGMENT_PASSES) {  // the observer's counters hold 15 passes
    const int seg_end = min(a.n_chunks, seg + 32 * ACC_SEGMENT_PASSES);
    SliceCounter c0, c1, c2, c3;  // disagreements of the new spin with neighbours 0..7, 8..15, (16..23, 24..31), bit-sliced
    for (int base = seg; base < seg_end; base += 32) {  // every lane runs every pass: the broadcasts are warp-wide
        const int ch = base + lane;
        const bool live = ch < a.n_chunks;
        uint32_t cfg[NH][4];
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int32_t nbj = __shfl_sync(0xffffffffu, tnb, 8 * h + j);
                v[j] = make_uint4(0, 0, 0, 0);
                if (nbj >= 0 && live) v[j] = __ldg(reinterpret_cast<const uint4*>(a.spin + static_cast<int64_t>(nbj) * a.ld) + ch);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) cfg[h][q] = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                cfg[h][0] += v[j].x << j;
                cfg[h][1] += v[j].y << j;
                cfg[h][2] += v[j].z << j;
                cfg[h][3] += v[j].w << j;
            }
        }
        uint32_t o[4];
        bool close = false;  // some draw of this pass is inside the window (or not a number: non-finite weights)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const U4 r = philox4x32_10_rk(static_cast<uint32_t>(node), a.chain_word0 + 4u * ch + q, 0u, TAG_SPIN, a.rk);
            const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
            o[q] = 0;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float d = split_screen<NH>(tab, cfg, q, c, rr[c]);
                close |= !(fabsf(d) > margin);
                o[q] |= (__float_as_uint(d) >> 31) << (8 * c);
            }
        }
        if (live && close) {
#pragma unroll 1
            for (int q = 0; q < 4; ++q) {
                const U4 r = philox4x32_10_rk(static_cast<uint32_t>(node), a.chain_word0 + 4u * ch + q, 0u, TAG_SPIN, a.rk);
                const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float d = split_screen<NH>(tab, cfg, q, c, rr[c]);
                    if (!(fabsf(d) > margin)) {
                        const float gamma = exact_seq_gamma(a, node, 16 * static_cast<int64_t>(ch) + 4 * q + c);
                        o[q] = (o[q] & ~(1u << (8 * c))) | ((exact_spin_draw(gamma, rr[c]) ? 1u : 0u) << (8 * c));
                    }
                }
            }
        }
        if (live) reinterpret_cast<uint4*>(drow)[ch] = make_uint4(o[0], o[1], o[2], o[3]);
        if (ACC && (own | static_cast<uint32_t>(row1 >= 0))) {
            if (16 * static_cast<int64_t>(ch + 1) > a.n_chains) {  // ragged last chunk or an idle lane: drop chains that do not exist
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t vm = live ? valid_mask(a.n_chains, ch, q) : 0u;
                    o[q] &= vm;
#pragma unroll
                    for (int h = 0; h < NH; ++h) cfg[h][q] &= vm;
                }
            }
            const uint32_t f[4] = {o[0] * 255u, o[1] * 255u, o[2] * 255u, o[3] * 255u};
            // bit j of a byte: neighbour 8 h + j differs from the new spin
            c0.add4(cfg[0][0] ^ f[0], cfg[0][1] ^ f[1], cfg[0][2] ^ f[2], cfg[0][3] ^ f[3]);
            c1.add4(cfg[1][0] ^ f[0], cfg[1][1] ^ f[1], cfg[1][2] ^ f[2], cfg[1][3] ^ f[3]);
            if (NH == 4) {
                c2.add4(cfg[NH - 2][0] ^ f[0], cfg[NH - 2][1] ^ f[1], cfg[NH - 2][2] ^ f[2], cfg[NH - 2][3] ^ f[3]);
                c3.add4(cfg[NH - 1][0] ^ f[0], cfg[NH - 1][1] ^ f[1], cfg[NH - 1][2] ^ f[2], cfg[NH - 1][3] ^ f[3]);
            }
            ones_total += __popc(o[0] + (o[1] << 1) + (o[2] << 2) + (o[3] << 3));
        }
    }
    if (ACC) {
        for (uint32_t left = own; left; left &= left - 1) {  // uniform over the warp
            const int e = __ffs(left) - 1;
            const int rank = __popc(tails & ((1u << e) - 1u));  // the entry's bit in the configuration
            uint32_t mine_here = rank < 8 ? c0.total(rank) : c1.total(rank & 7);
            if (NH == 4 && rank >= 16) mine_here = rank < 24 ? c2.total(rank & 7) : c3.total(rank & 7);
            const uint32_t t = __reduce_add_sync(0xffffffffu, mine_here);
            if (lane == e) mine += t;
        }
    }
    }
    if (ACC) {
        if (my_row >= 0) a.sums[my_row] += a.n_chains - 2ll * mine;
        if (row1 >= 0) {
            ones_total = __reduce_add_sync(0xffffffffu, ones_total);
            if (lane == 0) a.sums[row1] += 2ll * ones_total - a.n_chains;
        }
    }
}
// A sequential-sum node by whichever of the two routes its block prepared for it.
// WIDE: the block has nodes with four tables (more than 16 neighbours).  Blocks without them run the instantiation that
// does not carry that code (fewer spilled registers, half the shared memory).
template <bool ACC, bool WIDE>
__device__ __forceinline__ void seq_or_split_update(const SeqArgs& a, float* tab, int node) {
    const int32_t code = a.split_row ? __ldg(a.split_row + node) : -1;
    if (code < 0) seq_node_update<ACC>(a, node);
    else if (WIDE && (code & 1)) split_node_update<ACC, 4>(a, tab, node, code >> 1);
    else split_node_update<ACC, 2>(a, tab, node, code >> 1);
}
template <bool ACC, bool WIDE>
__global__ void __launch_bounds__(256, ACC && WIDE ? 3 : 4) k_spin_seq(const __grid_constant__ SeqArgs a) {
    __shared__ float s_tab[8][WIDE ? SPLIT_TAB : SPLIT_TAB / 2];
    for (int node = take_node(a); node >= 0; node = take_node(a)) seq_or_split_update<ACC, WIDE>(a, s_tab[threadIdx.x >> 5], node);
}

// Blocks that mix the two kinds of node: those with at most 8 neighbour slots take the threshold-table update, the
// others the sequential sum, warp by warp (a sparse random graph has a few high-degree nodes in every block; they
// should not cost the other nodes their tables).  lut_row[node] >= 0 is the node's row in the block's compact
// neighbour-list and table arrays, -1 marks a sequential-sum node.  The observer's pair-row map has SEQ_MAX entries
// per node for both kinds (a table node uses the first 8, indexed by neighbour slot).
struct HybridArgs {
    LutArgs lut;
    SeqArgs seq;
    const int32_t* lut_row;
};
template <bool ACC, bool WIDE>
__global__ void __launch_bounds__(256, ACC && WIDE ? 3 : 4) k_spin_hybrid(const __grid_constant__ HybridArgs a) {
    __shared__ uint32_t s_tab[8][WIDE ? SPLIT_TAB : SPLIT_TAB / 2];  // a warp's threshold table (256 words) or its two or four field tables
    for (int node = take_node(a.seq); node >= 0; node = take_node(a.seq)) {
        const int32_t row = __ldg(a.lut_row + node);
        if (row >= 0) lut_node_update<ACC, false>(a.lut, s_tab[threadIdx.x >> 5], node, row, static_cast<int64_t>(node) * SEQ_MAX);
        else seq_or_split_update<ACC, WIDE>(a.seq, reinterpret_cast<float*>(s_tab[threadIdx.x >> 5]), node);
    }
}

// Threshold-table update on a BIT-PACKED spin state (one bit per node and chain: word w of a row holds chains 32 w .. 32 w + 31),
// the same function of the same noise as k_spin_lut, so the states are the same bits.  One warp per node; a lane takes one
// word of each of the 8 neighbour rows (32 chains; the warp reads 128 contiguous bytes per row), transposes the 8 x 32 bit
// matrix into 32 configuration bytes (byte permutes to collect 8 x 8 blocks, three masked-shift steps to transpose each),
// looks the thresholds up in the node's table (staged in shared memory once per node) and compares them with the Philox
// words of the four-chain groups.  1.125 bytes of state per update instead of 9, at about the instruction count of the
// byte kernel: this kernel is bound by instruction issue, not by HBM.
// ACC: the fused moment observer; pair rows are population counts of XORed words.
struct PackedArgs {
    const int32_t* nbr;   // [n][8] global spin positions, -1 = unused slot
    const uint32_t* lut;  // [n][256]
    const uint32_t* src;  // packed rows of the spin class
    uint32_t* dst;        // first packed row of the block
    int64_t pw;           // words per packed row
    int32_t n;
    int32_t n_words;      // words that hold chains: ceil(n_chains / 32)
    uint32_t chain_word0;
    int64_t n_chains;
    PhiloxRoundKeys rk;
    const int32_t* m1_row;
    const int32_t* m2_row;
    long long* sums;
};
// 8 x 8 bit transpose of the matrix held as bytes of (lo, hi): bit b of byte i becomes bit i of byte b.
__device__ __forceinline__ void transpose_8x8(uint32_t& lo, uint32_t& hi) {
    uint32_t t;
    t = (lo ^ (lo << 7)) & 0x55005500u; lo ^= t ^ (t >> 7);
    t = (hi ^ (hi << 7)) & 0x55005500u; hi ^= t ^ (t >> 7);
    t = (lo ^ (lo << 14)) & 0x33330000u; lo ^= t ^ (t >> 14);
    t = (hi ^ (hi << 14)) & 0x33330000u; hi ^= t ^ (t >> 14);
    t = (hi ^ (lo >> 4)) & 0x0f0f0f0fu; hi ^= t; lo ^= t << 4;
}
template <bool ACC>
__global__ void __launch_bounds__(256, 4) k_packed_lut(const __grid_constant__ PackedArgs a) {
    __shared__ uint32_t s_lut[8][LUT_SIZE];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t* tab = s_lut[warp];
    for (int node = blockIdx.x * 8 + warp; node < a.n; node += gridDim.x * 8) {
        __syncwarp();  // the previous node's lookups are done
        const uint4* src = reinterpret_cast<const uint4*>(a.lut + static_cast<int64_t>(node) * LUT_SIZE);
        {  // the table is staged complemented: draw > threshold  <=>  draw + ~threshold carries out of 32 bits
            const uint4 q0 = __ldg(src + lane), q1 = __ldg(src + lane + 32);
            reinterpret_cast<uint4*>(tab)[lane] = make_uint4(~q0.x, ~q0.y, ~q0.z, ~q0.w);
            reinterpret_cast<uint4*>(tab)[lane + 32] = make_uint4(~q1.x, ~q1.y, ~q1.z, ~q1.w);
        }
        const int32_t nb = lane < LUT_BITS ? __ldg(a.nbr + static_cast<int64_t>(node) * LUT_BITS + lane) : -1;
        int32_t my_row = -1, row1 = -1;
        uint32_t own = 0, mine = 0, ones_total = 0;
        if (ACC) {
            my_row = lane < LUT_BITS ? __ldg(a.m2_row + static_cast<int64_t>(node) * LUT_BITS + lane) : -1;
            row1 = __ldg(a.m1_row + node);
            own = __ballot_sync(0xffffffffu, my_row >= 0);
        }
        __syncwarp();
        uint32_t* drow = a.dst + static_cast<int64_t>(node) * a.pw;
        for (int base = 0; base < a.n_words; base += 32) {  // every lane runs every pass: the broadcasts are warp-wide
            const int word = base + lane;
            const bool live = word < a.n_words;
            uint32_t w[LUT_BITS];
#pragma unroll
            for (int j = 0; j < LUT_BITS; ++j) {
                const int32_t nbj = __shfl_sync(0xffffffffu, nb, j);
                w[j] = (nbj >= 0 && live) ? __ldg(a.src + static_cast<int64_t>(nbj) * a.pw + word) : 0u;
            }
            // configuration bytes of the 32 chains: idx[g] holds chains 4 g .. 4 g + 3
            uint32_t idx[8];
            {
                const uint32_t a0 = __byte_perm(w[0], w[1], 0x5140), a1 = __byte_perm(w[2], w[3], 0x5140);
                const uint32_t a2 = __byte_perm(w[0], w[1], 0x7362), a3 = __byte_perm(w[2], w[3], 0x7362);
                const uint32_t b0 = __byte_perm(w[4], w[5], 0x5140), b1 = __byte_perm(w[6], w[7], 0x5140);
                const uint32_t b2 = __byte_perm(w[4], w[5], 0x7362), b3 = __byte_perm(w[6], w[7], 0x7362);
                idx[0] = __byte_perm(a0, a1, 0x5410); idx[1] = __byte_perm(b0, b1, 0x5410);
                idx[2] = __byte_perm(a0, a1, 0x7632); idx[3] = __byte_perm(b0, b1, 0x7632);
                idx[4] = __byte_perm(a2, a3, 0x5410); idx[5] = __byte_perm(b2, b3, 0x5410);
                idx[6] = __byte_perm(a2, a3, 0x7632); idx[7] = __byte_perm(b2, b3, 0x7632);
#pragma unroll
                for (int q = 0; q < 4; ++q) transpose_8x8(idx[2 * q], idx[2 * q + 1]);
            }
            // Chains 31 down to 0: each comparison is an add whose carry (draw > threshold: the spin becomes 0) is shifted into
            // the word by an add-with-carry, two integer operations per chain; the word is inverted at the end.
            uint32_t out = 0;
#pragma unroll
            for (int g = 7; g >= 0; --g) {
                const U4 r = philox4x32_10_rk(static_cast<uint32_t>(node), a.chain_word0 + 8u * static_cast<uint32_t>(word) + g, 0u, TAG_SPIN, a.rk);
                const uint32_t c = idx[g];
                const uint32_t t0 = tab[c & 0xffu], t1 = tab[(c >> 8) & 0xffu], t2 = tab[(c >> 16) & 0xffu], t3 = tab[c >> 24];
                uint32_t scratch;
                asm("add.cc.u32 %1, %2, %3;\n\taddc.u32 %0, %0, %0;" : "+r"(out), "=r"(scratch) : "r"(t3), "r"(r.w));
                asm("add.cc.u32 %1, %2, %3;\n\taddc.u32 %0, %0, %0;" : "+r"(out), "=r"(scratch) : "r"(t2), "r"(r.z));
                asm("add.cc.u32 %1, %2, %3;\n\taddc.u32 %0, %0, %0;" : "+r"(out), "=r"(scratch) : "r"(t1), "r"(r.y));
                asm("add.cc.u32 %1, %2, %3;\n\taddc.u32 %0, %0, %0;" : "+r"(out), "=r"(scratch) : "r"(t0), "r"(r.x));
            }
            out = ~out;
            const int64_t left = a.n_chains - 32 * static_cast<int64_t>(word);
            const uint32_t vm = !live || left <= 0 ? 0u : (left >= 32 ? 0xffffffffu : ((1u << static_cast<int>(left)) - 1u));
            out &= vm;  // chains past the last one stay 0
            if (live) drow[word] = out;
            if (ACC) {
                if (row1 >= 0) {
                    const uint32_t t = __reduce_add_sync(0xffffffffu, static_cast<uint32_t>(__popc(out)));
                    if (lane == 0) ones_total += t;
                }
#pragma unroll
                for (int j = 0; j < LUT_BITS; ++j) {
                    if (!((own >> j) & 1u)) continue;  // uniform over the warp
                    const uint32_t t = __reduce_add_sync(0xffffffffu, static_cast<uint32_t>(__popc((w[j] ^ out) & vm)));
                    if (lane == j) mine += t;
                }
            }
        }
        if (ACC) {
            if (my_row >= 0) a.sums[my_row] += a.n_chains - 2ll * mine;
            if (lane == 0 && row1 >= 0) a.sums[row1] += 2ll * ones_total - a.n_chains;
        }
    }
}

// Spin update for blocks the threshold-table and sequential-sum kernels cannot take: slots whose tail is a product of up to
// three spins, and slots with a categorical tail that selects the weight (spin_gibbs.rs:527-582).  Same states as
// k_spin_generic<0>, organised like k_spin_seq: one warp per node, 16 chains per lane per pass, one 16-byte load per
// neighbour row.  Lane e holds entry e of the node's list (its table and slot, in the canonical order) and fetches that
// entry's tail positions and weight once; the entry loop broadcasts them.  The product of the spin tails is the XOR of
// their sign bits; a categorical tail costs one weight lookup per chain.  Weights are read from the slot tables
// themselves, so a weight refresh needs no rebuild.  The sigmoid is screened as in k_spin_seq.
constexpr int WIDE_SPIN_TAILS = 3;
struct WideArgs {
    const DevTable* tabs;
    const int32_t* ent;     // [n][SEQ_MAX]: table << 24 | slot of the node's active slots in canonical order, -1 = none
    const uint32_t* first;  // [n] bit e: entry e is the first of its table
    const int32_t* cnt;     // [n]
    const uint8_t* spin;
    const uint8_t* cat;
    uint8_t* dst;
    int64_t ld;
    int32_t n;
    int32_t n_chunks;  // ld / 16
    uint32_t chain_word0;
    int64_t n_chains;
    PhiloxRoundKeys rk;
};
template <bool CAT>
__global__ void __launch_bounds__(256, 3) k_spin_wide(const __grid_constant__ WideArgs a) {
    const int lane = threadIdx.x & 31;
    const uint4 zeros = make_uint4(0, 0, 0, 0);
    for (int node = blockIdx.x * 8 + (threadIdx.x >> 5); node < a.n; node += gridDim.x * 8) {
        const int32_t code = __ldg(a.ent + static_cast<int64_t>(node) * SEQ_MAX + lane);
        const uint32_t first = __ldg(a.first + node);
        const int cnt = __ldg(a.cnt + node);
        int32_t nb0 = -1, nb1 = -1, nb2 = -1, nbc = -1, wdim = 1;
        float wv = 0.0f;
        const float* wp = nullptr;
        if (code >= 0) {
            const DevTable& T = a.tabs[code >> 24];
            const int64_t flat = static_cast<int64_t>(node) * T.k + (code & 0xffffff);
            if (T.n_spin > 0) nb0 = __ldg(T.idx[0] + flat);
            if (T.n_spin > 1) nb1 = __ldg(T.idx[1] + flat);
            if (T.n_spin > 2) nb2 = __ldg(T.idx[2] + flat);
            wp = T.w + flat * T.wdim;
            wdim = T.wdim;
            if (CAT && T.n_tails > T.n_spin) nbc = __ldg(T.idx[T.n_spin] + flat);
            else wv = __ldg(wp);
        }
        uint8_t* drow = a.dst + static_cast<int64_t>(node) * a.ld;
        for (int base = 0; base < a.n_chunks; base += 32) {  // every lane runs every pass: the entry broadcasts are warp-wide
            const int ch = base + lane;
            const bool live = ch < a.n_chunks;
            float gam[16], part[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) gam[i] = part[i] = 0.0f;
            auto sign_row = [&](int32_t nb) {  // bit 0 of a byte: that chain's spin is -1
                if (nb < 0 || !live) return zeros;
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(a.spin + static_cast<int64_t>(nb) * a.ld) + ch);
                return make_uint4(v.x ^ 0x01010101u, v.y ^ 0x01010101u, v.z ^ 0x01010101u, v.w ^ 0x01010101u);
            };
            for (int e = 0; e < cnt; ++e) {  // uniform over the warp
                const uint4 s0 = sign_row(__shfl_sync(0xffffffffu, nb0, e));
                const uint4 s1 = sign_row(__shfl_sync(0xffffffffu, nb1, e));
                const uint4 s2 = sign_row(__shfl_sync(0xffffffffu, nb2, e));
                const int32_t nce = CAT ? __shfl_sync(0xffffffffu, nbc, e) : -1;
                const float we = __shfl_sync(0xffffffffu, wv, e);
                if ((first >> e) & 1u) {  // a new table: close the previous one
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        gam[i] = __fadd_rn(gam[i], part[i]);
                        part[i] = 0.0f;
                    }
                }
                // +-1.0f per chain from the sign bit with one byte permute, as in k_spin_seq
                const uint32_t t[4] = {((s0.x ^ s1.x ^ s2.x) << 7) | 0x3f3f3f3fu, ((s0.y ^ s1.y ^ s2.y) << 7) | 0x3f3f3f3fu,
                                       ((s0.z ^ s1.z ^ s2.z) << 7) | 0x3f3f3f3fu, ((s0.w ^ s1.w ^ s2.w) << 7) | 0x3f3f3f3fu};
                if (CAT && nce >= 0) {  // the neighbour's category selects the weight; out of range selects none
                    const uint64_t wpe = __shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(wp), e);
                    const float* wrow = reinterpret_cast<const float*>(wpe);
                    const uint32_t wd = static_cast<uint32_t>(__shfl_sync(0xffffffffu, wdim, e));
                    uint4 xv = zeros;
                    if (live) xv = __ldg(reinterpret_cast<const uint4*>(a.cat + static_cast<int64_t>(nce) * a.ld) + ch);
                    const uint32_t x[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const uint32_t xi = (x[q] >> (8 * c)) & 0xffu;
                            const float wc = xi < wd ? __ldg(wrow + xi) : 0.0f;
                            const float sp = __uint_as_float(__byte_perm(t[q], 0x00800000u, 0x0654u | (c << 12)));
                            part[4 * q + c] = __fmaf_rn(sp, wc, part[4 * q + c]);
                        }
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const float sp = __uint_as_float(__byte_perm(t[q], 0x00800000u, 0x0654u | (c << 12)));
                            part[4 * q + c] = __fmaf_rn(sp, we, part[4 * q + c]);
                        }
                }
            }
            // d = 2^24 (u - p) with the approximate sigmoid; draws within 4e-6 of p are redone with the exact rule
            uint32_t o[4];
            float nearest = 16777216.0f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const U4 r = philox4x32_10_rk(static_cast<uint32_t>(node), a.chain_word0 + 4u * ch + q, 0u, TAG_SPIN, a.rk);
                const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
                o[q] = 0;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float gamma = __fadd_rn(gam[4 * q + c], part[4 * q + c]);
                    gam[4 * q + c] = gamma;
                    float ex, p24;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(gamma * -2.885390081777927f));
                    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(p24) : "f"(fmaf(ex, 5.9604644775390625e-8f, 5.9604644775390625e-8f)));  // 2^24 p
                    const float d = __uint2float_rn(rr[c] >> 8) - p24;
                    part[4 * q + c] = d;
                    nearest = fminf(nearest, fabsf(d));
                    o[q] |= (__float_as_uint(d) >> 31) << (8 * c);
                }
            }
            if (nearest <= 67.2f) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const U4 r = philox4x32_10_rk(static_cast<uint32_t>(node), a.chain_word0 + 4u * ch + q, 0u, TAG_SPIN, a.rk);
                    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (fabsf(part[4 * q + c]) <= 67.2f)
                            o[q] = (o[q] & ~(1u << (8 * c))) | ((exact_spin_draw(gam[4 * q + c], rr[c]) ? 1u : 0u) << (8 * c));
                }
            }
            if (live) {
                // chains past the last one stay 0, as every other kernel leaves them
#pragma unroll
                for (int q = 0; q < 4; ++q) o[q] &= valid_mask(a.n_chains, ch, q);
                reinterpret_cast<uint4*>(drow)[ch] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
}

// Chain-sliced variant for programs small enough that four chains of every spin fit in one CTA's shared memory.
// Chains never interact, so a CTA that owns chains 4q..4q+3 can run a whole schedule on its own: it loads one 32-bit
// word per spin (4 chains), walks the list of block updates with a CTA barrier after each, and stores the words back.
// No grid barrier, no launch per block.  One thread updates one node for the four chains with exactly one Philox call
// (the four output words are the four chains' draws), so the states are the bits the other kernels produce.
// The fused observer keeps signed per-row partial sums in shared memory (each row is owned by one node, hence by one
// thread) and adds them to the global sums once at the end.
struct SliceBlock {
    const int32_t* nbr;    // [n][8]
    const uint32_t* lut;   // [n][256]
    const int32_t* m1_row; // [n] or null
    const int32_t* m2_row; // [n][8] or null
    int32_t n;
    int32_t offset;        // first global spin position of the block
    int32_t lut_shift;     // resident copy: 2^lut_shift table entries per node (the block's largest neighbour count)
    int32_t smem_word;     // resident copy: first word of this block's tables in dynamic shared memory
};
struct SliceStep {
    int32_t block;
    int32_t acc;
    PhiloxRoundKeys rk;
};
static_assert(sizeof(SliceStep) == 88, "SliceStep is copied word by word");
constexpr int SLICE_MAX_BLOCKS = 32;
struct SliceArgs {
    const SliceBlock* blocks;
    const SliceStep* steps;
    int32_t n_blocks;
    int32_t n_steps;
    int32_t n_spin;    // spins of the class (free and clamped)
    int32_t n_rows;    // observer rows (0 without observer)
    int32_t resident;  // 1: neighbour lists, the reachable part of the threshold tables and the observer's row maps are copied to shared memory first
    uint32_t chain_word0;
    uint8_t* spin;
    int64_t ld;
    int64_t n_chains;
    unsigned long long* sums;
};
constexpr int SLICE_STEP_WORDS = sizeof(SliceStep) / 4;
// words of dynamic shared memory a block's resident tables take: neighbours, compact thresholds, observer row maps
// (rounded to 16 bytes; the two arrays read with 16-byte loads come first)
inline int64_t slice_block_words(int64_t n, int lut_shift, bool acc) {
    const int64_t n_pad = (n + 31) / 32 * 32;
    return (n * LUT_BITS + (n_pad << lut_shift) + (acc ? n * (1 + LUT_BITS) : 0) + 3) / 4 * 4;
}

// RESIDENT: neighbour lists, the reachable part of the threshold tables and the observer's row maps are copied into
// shared memory first (word offsets into s_dyn; thresholds entry-major with a node stride that is a multiple of 32, so
// consecutive nodes hit distinct banks whatever their configurations); otherwise they are read from global memory.
struct SliceView {
    const int32_t* nbr;
    const uint32_t* lut;
    const int32_t* m1;
    const int32_t* m2;
    int32_t nbr_w, lut_w, m1_w, m2_w;  // resident: first words in s_dyn (m1_w < 0: no observer rows)
    int32_t n, offset, n_pad;
    int32_t deg;  // largest neighbour count in the block: slots from deg on are empty for every node
};
template <bool RESIDENT>
__global__ void __launch_bounds__(512) k_spin_lut_sliced(const __grid_constant__ SliceArgs a) {
    extern __shared__ __align__(16) uint32_t s_dyn[];
    __shared__ SliceStep s_step[2];
    __shared__ SliceView s_blk[SLICE_MAX_BLOCKS];
    uint32_t* st = s_dyn;                                          // [n_spin]
    int32_t* part = reinterpret_cast<int32_t*>(s_dyn + a.n_spin);  // [n_rows]
    const int32_t* sw = reinterpret_cast<const int32_t*>(s_dyn);
    const int tid = threadIdx.x, T = blockDim.x;
    const int quad = blockIdx.x;
    const int64_t remaining = a.n_chains - 4ll * quad;
    const int left = remaining >= 4 ? 4 : static_cast<int>(remaining);  // chains of this slice that exist
    const uint32_t vm = left >= 4 ? 0xffffffffu : (0xffffffffu >> (8 * (4 - left)));
    for (int i = tid; i < a.n_spin; i += T) st[i] = *reinterpret_cast<const uint32_t*>(a.spin + static_cast<int64_t>(i) * a.ld + 4 * quad);
    for (int i = tid; i < a.n_rows; i += T) part[i] = 0;
    if (tid < SLICE_STEP_WORDS) reinterpret_cast<uint32_t*>(&s_step[0])[tid] = __ldg(reinterpret_cast<const uint32_t*>(a.steps) + tid);
    if (tid < a.n_blocks) {
        const SliceBlock b = a.blocks[tid];
        SliceView v;
        v.nbr = b.nbr; v.lut = b.lut; v.m1 = b.m1_row; v.m2 = b.m2_row;
        v.n = b.n; v.offset = b.offset; v.n_pad = (b.n + 31) / 32 * 32;
        v.deg = b.lut_shift;
        v.nbr_w = b.smem_word;
        v.m2_w = v.nbr_w + b.n * LUT_BITS;
        v.lut_w = b.m1_row ? v.m2_w + b.n * LUT_BITS : v.m2_w;
        v.m1_w = b.m1_row ? v.lut_w + (v.n_pad << b.lut_shift) : -1;
        s_blk[tid] = v;
    }
    __syncthreads();
    if (RESIDENT) {
        for (int bi = 0; bi < a.n_blocks; ++bi) {
            const SliceView& v = s_blk[bi];
            const int shift = a.blocks[bi].lut_shift, per = 1 << shift;
            int32_t* w = reinterpret_cast<int32_t*>(s_dyn);
            for (int i = tid; i < v.n * LUT_BITS; i += T) w[v.nbr_w + i] = __ldg(v.nbr + i);
            for (int i = tid; i < v.n * per; i += T) {
                const int node = i >> shift, c = i & (per - 1);
                s_dyn[v.lut_w + c * v.n_pad + node] = __ldg(v.lut + static_cast<int64_t>(node) * LUT_SIZE + c);
            }
            if (v.m1_w >= 0) {
                for (int i = tid; i < v.n; i += T) w[v.m1_w + i] = __ldg(v.m1 + i);
                for (int i = tid; i < v.n * LUT_BITS; i += T) w[v.m2_w + i] = __ldg(v.m2 + i);
            }
        }
        __syncthreads();
    }
    for (int32_t i = 0; i < a.n_steps; ++i) {
        const SliceStep& sp = s_step[i & 1];
        const SliceView& v = s_blk[sp.block];
        const int32_t n = v.n;
        const bool acc = sp.acc != 0;
        const bool wide = v.deg > 4;  // uniform over the CTA: blocks of degree <= 4 (lattices) skip the upper four slots
        for (int node = tid; node < n; node += T) {
            int4 n0, n1 = make_int4(-1, -1, -1, -1);
            if (RESIDENT) {
                n0 = *reinterpret_cast<const int4*>(sw + v.nbr_w + node * LUT_BITS);
                if (wide) n1 = *reinterpret_cast<const int4*>(sw + v.nbr_w + node * LUT_BITS + 4);
            } else {
                n0 = __ldg(reinterpret_cast<const int4*>(v.nbr + static_cast<int64_t>(node) * LUT_BITS));
                if (wide) n1 = __ldg(reinterpret_cast<const int4*>(v.nbr + static_cast<int64_t>(node) * LUT_BITS) + 1);
            }
            uint32_t cfg = 0;
            if (n0.x >= 0) cfg += st[n0.x];
            if (n0.y >= 0) cfg += st[n0.y] << 1;
            if (n0.z >= 0) cfg += st[n0.z] << 2;
            if (n0.w >= 0) cfg += st[n0.w] << 3;
            if (wide) {
                if (n1.x >= 0) cfg += st[n1.x] << 4;
                if (n1.y >= 0) cfg += st[n1.y] << 5;
                if (n1.z >= 0) cfg += st[n1.z] << 6;
                if (n1.w >= 0) cfg += st[n1.w] << 7;
            }
            uint32_t t0, t1, t2, t3;
            if (RESIDENT) {  // configuration bytes stay below 2^(neighbour count), inside the copied part of the table
                const uint32_t* L = s_dyn + v.lut_w + node;
                t0 = L[(cfg & 0xffu) * v.n_pad];
                t1 = L[((cfg >> 8) & 0xffu) * v.n_pad];
                t2 = L[((cfg >> 16) & 0xffu) * v.n_pad];
                t3 = L[(cfg >> 24) * v.n_pad];
            } else {
                const uint32_t* L = v.lut + static_cast<int64_t>(node) * LUT_SIZE;
                t0 = __ldg(L + (cfg & 0xffu));
                t1 = __ldg(L + ((cfg >> 8) & 0xffu));
                t2 = __ldg(L + ((cfg >> 16) & 0xffu));
                t3 = __ldg(L + (cfg >> 24));
            }
            // the step's keys live in shared memory here: two loads and the per-round adds are cheaper than twenty loads
            const U4 r = philox4x32_10(static_cast<uint32_t>(node), a.chain_word0 + static_cast<uint32_t>(quad), 0u, TAG_SPIN, sp.rk.k0[0], sp.rk.k1[0]);
            uint32_t o = (r.x <= t0) ? 1u : 0u;
            o |= (r.y <= t1) ? 0x100u : 0u;
            o |= (r.z <= t2) ? 0x10000u : 0u;
            o |= (r.w <= t3) ? 0x1000000u : 0u;
            st[v.offset + node] = o;  // neighbours are never in the block being updated, so nobody reads this word before the barrier
            if (acc && v.m1_w >= 0) {
                int32_t row1;
                int4 r0, r1 = make_int4(-1, -1, -1, -1);
                if (RESIDENT) {
                    row1 = sw[v.m1_w + node];
                    r0 = *reinterpret_cast<const int4*>(sw + v.m2_w + node * LUT_BITS);
                    if (wide) r1 = *reinterpret_cast<const int4*>(sw + v.m2_w + node * LUT_BITS + 4);
                } else {
                    row1 = __ldg(v.m1 + node);
                    r0 = __ldg(reinterpret_cast<const int4*>(v.m2 + static_cast<int64_t>(node) * LUT_BITS));
                    if (wide) r1 = __ldg(reinterpret_cast<const int4*>(v.m2 + static_cast<int64_t>(node) * LUT_BITS) + 1);
                }
                if (row1 >= 0) part[row1] += 2 * __popc(o & vm) - left;
                const uint32_t d = (cfg ^ (o * 255u)) & vm;  // bit j of a byte: neighbour j differs from the new spin
                if (r0.x >= 0) part[r0.x] += left - 2 * __popc(d & 0x01010101u);
                if (r0.y >= 0) part[r0.y] += left - 2 * __popc(d & 0x02020202u);
                if (r0.z >= 0) part[r0.z] += left - 2 * __popc(d & 0x04040404u);
                if (r0.w >= 0) part[r0.w] += left - 2 * __popc(d & 0x08080808u);
                if (wide) {
                    if (r1.x >= 0) part[r1.x] += left - 2 * __popc(d & 0x10101010u);
                    if (r1.y >= 0) part[r1.y] += left - 2 * __popc(d & 0x20202020u);
                    if (r1.z >= 0) part[r1.z] += left - 2 * __popc(d & 0x40404040u);
                    if (r1.w >= 0) part[r1.w] += left - 2 * __popc(d & 0x80808080u);
                }
            }
        }
        if (i + 1 < a.n_steps && tid < SLICE_STEP_WORDS)
            reinterpret_cast<uint32_t*>(&s_step[(i + 1) & 1])[tid] = __ldg(reinterpret_cast<const uint32_t*>(a.steps + i + 1) + tid);
        __syncthreads();
    }
    for (int i = tid; i < a.n_spin; i += T) *reinterpret_cast<uint32_t*>(a.spin + static_cast<int64_t>(i) * a.ld + 4 * quad) = st[i];
    for (int i = tid; i < a.n_rows; i += T)
        if (part[i] != 0) atomicAdd(a.sums + i, static_cast<unsigned long long>(static_cast<long long>(part[i])));
}
