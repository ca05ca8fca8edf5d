// Implicit 3-D periodic Potts-like lattice: K categories per node, one K x K interaction table per lattice direction
// (shared by every edge of that direction), per-node unary terms, two checkerboard blocks, Gumbel-argmax updates.
//
// Semantics = FactorSamplingProgram (crates/thrml-models/src/factor.rs:153-184) over the factors
//   CategoricalEBMFactor([all nodes], unary[N,K,1]),
//   CategoricalEBMFactor([U, U + e_d], T_d broadcast to [N,K,K])  for d = x, y, z            (discrete_ebm.rs:792-851)
// with blocks [(x+y+z) even, (x+y+z) odd] and CategoricalGibbsConditional (softmax.rs:228-271, 586-709): a node's logits are
//   theta[c] = unary[c] + Tx[c][s(+x)] + Tx[s(-x)][c] + Ty[c][s(+y)] + Ty[s(-y)][c] + Tz[c][s(+z)] + Tz[s(-z)][c]
// added left to right in f32 — the order in which the reference's per-block tables (each with one slot) are summed — so
// the sampled states equal the explicit program's bit for bit, without its [N,6,K*K] weight tensors (2.5 GB per block at
// 128^3, K = 10).  Node index = (x*ny + y)*nz + z; state = one byte per node and chain, chains innermost.
#include <algorithm>
#include <cmath>
#include <memory>
#include <vector>

#include "comm.h"
#include "ctx.h"
#include "devbuf.h"
#include "device_math.cuh"

using namespace thrml;

namespace {

constexpr int MAX_K = 32;

struct PottsArgs {
    uint8_t* state;        // [N][ld]
    const float* tables;   // [3][K][K], beta already applied
    const float* unary;    // [N][K], beta already applied
    int32_t nx, ny, nz, K, colour;
    int64_t ld, n_chains;
    uint32_t chain_word0, k0, k1;
    const float* pair_tables;  // [3][K][K][K]: P_d[c][s_plus][s_minus] = T_d[c][s_plus] + T_d[s_minus][c] rounded once (PAIR kernels only)
    float table_mag;           // 2 (max|T_x| + max|T_y| + max|T_z|): bound of the six table terms of a field
    int32_t* counts;           // [N][K] category counts to add this update's draws to, or null (K <= 16 only)
};

// Exact Gumbel-argmax of one chain (byte `sh / 8` of the neighbour words): the rule of softmax.rs:60-97 with the
// deterministic logarithm.  Kept out of line: the update kernel calls it for about one update in 10^4.
__device__ __noinline__ uint32_t potts_exact_argmax(const float* s_tab, const float* unary_row, int K, int sh, uint32_t px, uint32_t mx, uint32_t py, uint32_t my,
                                                    uint32_t pz, uint32_t mz, uint32_t in_block, uint32_t chain, uint32_t k0, uint32_t k1, bool quad_noise) {
    const int KK = K * K;
    float top = 0.f;
    uint32_t arg = 0;
    U4 rr;
    for (int cat = 0; cat < K; ++cat) {
        float th = __ldg(unary_row + cat);
        th = __fadd_rn(th, s_tab[cat * K + ((px >> sh) & 0xffu)]);
        th = __fadd_rn(th, s_tab[((mx >> sh) & 0xffu) * K + cat]);
        th = __fadd_rn(th, s_tab[KK + cat * K + ((py >> sh) & 0xffu)]);
        th = __fadd_rn(th, s_tab[KK + ((my >> sh) & 0xffu) * K + cat]);
        th = __fadd_rn(th, s_tab[2 * KK + cat * K + ((pz >> sh) & 0xffu)]);
        th = __fadd_rn(th, s_tab[2 * KK + ((mz >> sh) & 0xffu) * K + cat]);
        uint32_t word;
        if (quad_noise) {  // one call per category serves the four chains of a quad
            rr = philox4x32_10(in_block, chain >> 2, static_cast<uint32_t>(cat), TAG_CAT, k0, k1);
            word = pick(rr, chain & 3u);
        } else {
            if ((cat & 3) == 0) rr = philox4x32_10(in_block, chain, static_cast<uint32_t>(cat >> 2), TAG_CAT, k0, k1);
            word = pick(rr, cat & 3);
        }
        const float u = u23_open(word);
        const float p = __fadd_rn(th, -det_log(-det_log(u)));
        if (cat == 0 || p > top) { top = p; arg = cat; }
    }
    return arg;
}

// KT > 0: the category count as a compile-time constant.  The category loop then unrolls completely, which turns the
// table offsets cat * K and the choice of the Philox word into immediates (the integer pipe is the busy one here).
// PAIR: the screen reads one pre-added entry per direction, P_d[c][s_plus][s_minus], instead of two table entries: three
// lookups and adds per category and chain instead of six.  The re-associated field differs from the canonical one by at
// most 12 roundings of (|unary| + table_mag), which widens the window inside which the exact rule decides.
// CTAs stride over the colour's nodes (eight per pass), so the tables are staged once per CTA.
// QUAD: the engine's own key -> noise mapping (thrml_potts_set_noise): the uniform of (node, chain c, category k) is word c & 3
// of Philox(node, c >> 2, k, tag), so one call per category serves the thread's four chains (10 calls instead of 12 at K = 10).
template <int KT, bool PAIR, bool QUAD>
__global__ void __launch_bounds__(256, 3) k_potts_update(PottsArgs a) {
    extern __shared__ float s_tab[];  // [3][K][K], then (PAIR) [3][K][K][K]
    for (int i = threadIdx.x + threadIdx.y * blockDim.x; i < 3 * a.K * a.K; i += blockDim.x * blockDim.y) s_tab[i] = a.tables[i];
    if (PAIR)
        for (int i = threadIdx.x + threadIdx.y * blockDim.x; i < 3 * a.K * a.K * a.K; i += blockDim.x * blockDim.y) s_tab[3 * a.K * a.K + i] = a.pair_tables[i];
    __syncthreads();
    const int half_z = a.nz >> 1;
    const int64_t n_block = static_cast<int64_t>(a.nx) * a.ny * half_z;
    const int n_groups = static_cast<int>((a.ld + 127) / 128);  // a warp takes its node's chains 128 at a time
    // index among the nodes of this colour
    for (int64_t in_block = static_cast<int64_t>(blockIdx.x) * 8 + threadIdx.y; in_block < n_block; in_block += static_cast<int64_t>(gridDim.x) * 8) {
    unsigned long long cnt_lo = 0ull, cnt_hi = 0ull;  // a.counts: this lane's draws of the node, 8-bit fields per category
    for (int group = 0; group < n_groups; ++group) {
    const int quad = group * 32 + threadIdx.x;
    if (4 * static_cast<int64_t>(quad) >= a.ld) continue;  // never taken when the counts ride along (ld is a multiple of 128 then)
    const int zz = static_cast<int>(in_block % half_z);
    const int y = static_cast<int>((in_block / half_z) % a.ny);
    const int x = static_cast<int>(in_block / (static_cast<int64_t>(half_z) * a.ny));
    const int z = 2 * zz + ((x + y + a.colour) & 1);
    auto node_of = [&](int xx, int yy, int zz2) { return (static_cast<int64_t>(xx) * a.ny + yy) * a.nz + zz2; };
    auto word = [&](int64_t node) { return *reinterpret_cast<const uint32_t*>(a.state + node * a.ld + 4 * static_cast<int64_t>(quad)); };
    const int64_t node = node_of(x, y, z);
    const uint32_t px = word(node_of(x + 1 == a.nx ? 0 : x + 1, y, z)), mx = word(node_of(x == 0 ? a.nx - 1 : x - 1, y, z));
    const uint32_t py = word(node_of(x, y + 1 == a.ny ? 0 : y + 1, z)), my = word(node_of(x, y == 0 ? a.ny - 1 : y - 1, z));
    const uint32_t pz = word(node_of(x, y, z + 1 == a.nz ? 0 : z + 1)), mz = word(node_of(x, y, z == 0 ? a.nz - 1 : z - 1));
    const int K = KT > 0 ? KT : a.K, KK = K * K;
    auto theta = [&](int cat, int sh, float un) {
        float th = un;  // 0 + unary
        th = __fadd_rn(th, s_tab[cat * K + ((px >> sh) & 0xffu)]);            // this node is U of its +x edge: T[c][s_v]
        th = __fadd_rn(th, s_tab[((mx >> sh) & 0xffu) * K + cat]);            // and V of its -x edge: T[s_u][c]
        th = __fadd_rn(th, s_tab[KK + cat * K + ((py >> sh) & 0xffu)]);
        th = __fadd_rn(th, s_tab[KK + ((my >> sh) & 0xffu) * K + cat]);
        th = __fadd_rn(th, s_tab[2 * KK + cat * K + ((pz >> sh) & 0xffu)]);
        th = __fadd_rn(th, s_tab[2 * KK + ((mz >> sh) & 0xffu) * K + cat]);
        return th;
    };
    auto noise = [&](int c, int cat) {
        return philox4x32_10(static_cast<uint32_t>(in_block), 4u * (a.chain_word0 + static_cast<uint32_t>(quad)) + c, static_cast<uint32_t>(cat >> 2), TAG_CAT, a.k0, a.k1);
    };
    // First pass with fast logarithms.  The exact rule is argmax_c fl(theta_c - ln(-ln u_c)) with the deterministic
    // logarithm (softmax.rs:84) and the first maximum winning (gumbel_argmax/kernel.rs:81-83).  Here l = -ln u comes from
    // the hardware base-2 logarithm, whose absolute error (2^-22 in log2 u, 1.7e-7 in ln u) becomes a relative error of
    // 1.7e-7 / l in l and therefore an absolute error of 1.7e-7 / l in ln l; the outer logarithm adds at most 3.6e-6.  Each
    // score is within 4e-6 + 2e-7 / l of the exact one, so a leader more than 3 (4e-6 + 2e-7 / l_min) ahead of the runner-up
    // (l_min = the smallest l among the chain's categories) is the exact argmax.  Anything closer (about one update in 10^4)
    // is recomputed exactly for that chain.
    float best[4], second[4], lmin[4];
    uint32_t arg[4] = {0, 0, 0, 0};
    U4 r[4], rq;
    uint32_t ix[3][4];  // PAIR: s_plus * K + s_minus per direction and chain
    if (PAIR) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            ix[0][c] = ((px >> (8 * c)) & 0xffu) * K + ((mx >> (8 * c)) & 0xffu);
            ix[1][c] = ((py >> (8 * c)) & 0xffu) * K + ((my >> (8 * c)) & 0xffu);
            ix[2][c] = ((pz >> (8 * c)) & 0xffu) * K + ((mz >> (8 * c)) & 0xffu);
        }
    }
    float unmax = 0.0f;
#pragma unroll
    for (int cat = 0; cat < (KT > 0 ? KT : K); ++cat) {
        const float un = __ldg(a.unary + node * K + cat);
        if (PAIR) unmax = fmaxf(unmax, fabsf(un));
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float th;
            if (PAIR) {
                const float* pt = s_tab + 3 * KK + cat * KK;
                th = ((un + pt[ix[0][c]]) + pt[K * KK + ix[1][c]]) + pt[2 * K * KK + ix[2][c]];
            } else {
                th = theta(cat, 8 * c, un);
            }
            if (QUAD) { if (c == 0) rq = philox4x32_10(static_cast<uint32_t>(in_block), a.chain_word0 + static_cast<uint32_t>(quad), static_cast<uint32_t>(cat), TAG_CAT, a.k0, a.k1); }
            else if ((cat & 3) == 0) r[c] = noise(c, cat);
            const uint32_t word = QUAD ? pick(rq, c) : pick(r[c], cat & 3);
            // the 23-bit uniform (m + 0.5) 2^-23 of u23_open, formed exactly as (1 + m 2^-23) - (1 - 2^-24)
            const float u = __uint_as_float(0x3f800000u | (word >> 9)) - 0.99999994039535522461f;
            const float l1 = lg2_normal(u) * -0.6931471805599453f;  // -ln u > 0
            const float p = fmaf(lg2_normal(l1), -0.6931471805599453f, th);  // th - ln(l1)
            if (cat == 0) { best[c] = p; second[c] = -3.0e38f; lmin[c] = l1; }
            else {
                lmin[c] = fminf(lmin[c], l1);
                second[c] = fmaxf(second[c], fminf(best[c], p));  // runner-up: the smaller of the old leader and the newcomer, if it beats the old runner-up
                if (p > best[c]) { best[c] = p; arg[c] = cat; }
            }
        }
    }
    // each PAIR score is off by at most 12 x 2^-24 (|unary| + table_mag) more; twice that for leader and runner-up, and a third on top
    const float base = PAIR ? fmaf(2.0e-6f, unmax + a.table_mag, 1.2e-5f) : 1.2e-5f;
#pragma unroll
    for (int c = 0; c < 4; ++c)
        if (!(best[c] - second[c] > base + 6.0e-7f * rcp_normal(lmin[c])))
            arg[c] = potts_exact_argmax(s_tab, a.unary + node * K, K, 8 * c, px, mx, py, my, pz, mz, static_cast<uint32_t>(in_block),
                                        4u * (a.chain_word0 + static_cast<uint32_t>(quad)) + c, a.k0, a.k1, QUAD);
    uint32_t out = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c)
        if (4 * static_cast<int64_t>(quad) + c < a.n_chains) out |= arg[c] << (8 * c);
    *reinterpret_cast<uint32_t*>(a.state + node * a.ld + 4 * static_cast<int64_t>(quad)) = out;
    if (a.counts) {
        // Category marginals of the draws just made (the observation that follows the sweep sees exactly these values: a
        // node is updated once per sweep).  A lane counts its chains in 8-bit fields (categories 0-7 and 8-15 in two 64-bit
        // words; at most 4 per pass, 252 over the 63 passes the launch allows).
#pragma unroll
        for (int c = 0; c < 4; ++c)
            if (4 * static_cast<int64_t>(quad) + c < a.n_chains) {
                if (arg[c] < 8u) cnt_lo += 1ull << (8u * arg[c]);
                else cnt_hi += 1ull << (8u * (arg[c] - 8u));
            }
    }
    }
    if (a.counts) {
        // the warp adds its lanes' fields, widened to 16 bits (at most 32 x 252), and lane k adds category k's total to the
        // node's counter; the warp owns the node: no atomics
        const int Kc = KT > 0 ? KT : a.K;
        const uint32_t w4[4] = {static_cast<uint32_t>(cnt_lo), static_cast<uint32_t>(cnt_lo >> 32), static_cast<uint32_t>(cnt_hi), static_cast<uint32_t>(cnt_hi >> 32)};
        uint32_t total = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (4 * j >= Kc) break;  // uniform
            const uint32_t even = __reduce_add_sync(0xffffffffu, w4[j] & 0x00ff00ffu), odd = __reduce_add_sync(0xffffffffu, (w4[j] >> 8) & 0x00ff00ffu);
            const int k = static_cast<int>(threadIdx.x) - 4 * j;  // categories 4 j .. 4 j + 3 live in this word
            if (k >= 0 && k < 4) total = ((k & 1) ? odd : even) >> (16 * (k >> 1)) & 0xffffu;
        }
        if (static_cast<int>(threadIdx.x) < Kc) {
            const int zz = static_cast<int>(in_block % half_z);
            const int y = static_cast<int>((in_block / half_z) % a.ny);
            const int x = static_cast<int>(in_block / (static_cast<int64_t>(half_z) * a.ny));
            const int64_t node = (static_cast<int64_t>(x) * a.ny + y) * a.nz + 2 * zz + ((x + y + a.colour) & 1);
            a.counts[node * Kc + threadIdx.x] += static_cast<int32_t>(total);
        }
    }
    }
}

__global__ void __launch_bounds__(256) k_potts_randomize(uint8_t* state, int32_t nx, int32_t ny, int32_t nz, int32_t K, int32_t colour, int64_t ld, int64_t n_chains,
                                                        uint32_t chain_word0, uint32_t k0, uint32_t k1) {
    const int quad = blockIdx.y * 32 + threadIdx.x;
    const int64_t in_block = static_cast<int64_t>(blockIdx.x) * 8 + threadIdx.y;
    const int half_z = nz >> 1;
    if (in_block >= static_cast<int64_t>(nx) * ny * half_z || 4 * static_cast<int64_t>(quad) >= ld) return;
    const int zz = static_cast<int>(in_block % half_z), y = static_cast<int>((in_block / half_z) % ny), x = static_cast<int>(in_block / (static_cast<int64_t>(half_z) * ny));
    const int64_t node = (static_cast<int64_t>(x) * ny + y) * nz + 2 * zz + ((x + y + colour) & 1);
    const U4 r = philox4x32_10(static_cast<uint32_t>(in_block), chain_word0 + static_cast<uint32_t>(quad), 0u, TAG_RAND, k0, k1);
    uint32_t out = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c)
        if (4 * static_cast<int64_t>(quad) + c < n_chains) out |= static_cast<uint32_t>((static_cast<uint64_t>(pick(r, c) >> 8) * static_cast<uint64_t>(K)) >> 24) << (8 * c);
    *reinterpret_cast<uint32_t*>(state + node * ld + 4 * static_cast<int64_t>(quad)) = out;
}

// counts[node][category] += number of chains in that category (the category-marginal observer).
__global__ void __launch_bounds__(256) k_potts_marginals(const uint8_t* state, int64_t n_nodes, int32_t K, int64_t ld, int64_t n_chains, int32_t* counts) {
    const int64_t node = static_cast<int64_t>(blockIdx.x) * 8 + threadIdx.y;
    if (node >= n_nodes) return;
    int total = 0;  // lane k keeps the total of category k (K <= 32)
    for (int64_t base = 0; base < n_chains; base += 128) {
        const int64_t chain = base + 4 * threadIdx.x;
        uint32_t wd = 0xffffffffu;
        if (chain < n_chains) {
            wd = *reinterpret_cast<const uint32_t*>(state + node * ld + chain);
            const int64_t left = n_chains - chain;
            if (left < 4) wd |= 0xffffffffu << (8 * static_cast<int>(left));  // padding -> 0xff, matches no category
        }
        for (int k = 0; k < K; ++k) {
            const int c = ((wd & 0xffu) == static_cast<uint32_t>(k)) + (((wd >> 8) & 0xffu) == static_cast<uint32_t>(k)) + (((wd >> 16) & 0xffu) == static_cast<uint32_t>(k)) +
                          ((wd >> 24) == static_cast<uint32_t>(k));
            const int sum = __reduce_add_sync(0xffffffffu, c);
            if (threadIdx.x == k) total += sum;
        }
    }
    if (threadIdx.x < K) counts[node * K + threadIdx.x] += total;  // one warp owns the node: no atomics
}

// The same counts for K <= 10 and at most 2016 chains: a lane keeps the counts of all categories of its chains in one
// 64-bit word (ten 6-bit fields, at most 63 each), so the warp reduces once per category instead of once per category and
// 128 chains.  A warp takes two nodes per pass and issues every load (state rows and old counts) before it counts, so
// enough bytes are in flight to stream the state at memory speed.
__global__ void __launch_bounds__(256) k_potts_marginals_packed(const uint8_t* state, int64_t n_nodes, int32_t K, int64_t ld, int64_t n_chains, int32_t* counts) {
    constexpr int NODES = 2, PASSES = 4;  // 4 passes of 512 chains cover the 2016-chain limit
    const int lane = threadIdx.x;
    const int64_t node0 = (static_cast<int64_t>(blockIdx.x) * 8 + threadIdx.y) * NODES;
    if (node0 >= n_nodes) return;
    uint4 v[NODES][PASSES];
    int32_t old[NODES];
#pragma unroll
    for (int i = 0; i < NODES; ++i) {
        const int64_t node = node0 + i;
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int64_t chain = 16 * static_cast<int64_t>(lane) + 512 * p;
            v[i][p] = make_uint4(0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu);  // bytes that are no category: counted nowhere
            if (node < n_nodes && chain < n_chains) v[i][p] = *reinterpret_cast<const uint4*>(state + node * ld + chain);
        }
        old[i] = (node < n_nodes && lane < K) ? counts[node * K + lane] : 0;
    }
#pragma unroll
    for (int i = 0; i < NODES; ++i) {
        const int64_t node = node0 + i;
        if (node >= n_nodes) break;
        unsigned long long acc = 0ull;
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int64_t chain = 16 * static_cast<int64_t>(lane) + 512 * p;
            const int live = static_cast<int>(max(static_cast<int64_t>(0), min(static_cast<int64_t>(16), n_chains - chain)));  // the row's padding bytes are zero, not 0xff
            const uint32_t wds[4] = {v[i][p].x, v[i][p].y, v[i][p].z, v[i][p].w};
#pragma unroll
            for (int b = 0; b < 16; ++b)
                if (b < live) acc += 1ull << (6u * min((wds[b >> 2] >> (8 * (b & 3))) & 0xffu, 10u));
        }
        int32_t mine = 0;
        for (int k = 0; k < K; ++k) {
            const int sum = __reduce_add_sync(0xffffffffu, static_cast<int>((acc >> (6 * k)) & 63ull));
            if (lane == k) mine = sum;
        }
        if (lane < K) counts[node * K + lane] = old[i] + mine;  // one warp owns the node: no atomics
    }
}

__global__ void k_potts_transpose_in(const uint8_t* src, uint8_t* dst, int64_t n, int64_t n_chains, int64_t ld) {
    __shared__ uint8_t tile[32][33];
    const int64_t node0 = static_cast<int64_t>(blockIdx.x) * 32, chain0 = static_cast<int64_t>(blockIdx.y) * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int64_t chain = chain0 + r, node = node0 + threadIdx.x;
        tile[r][threadIdx.x] = (chain < n_chains && node < n) ? src[chain * n + node] : 0;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int64_t node = node0 + r, chain = chain0 + threadIdx.x;
        if (node < n && chain < ld) dst[node * ld + chain] = chain < n_chains ? tile[threadIdx.x][r] : 0;
    }
}
__global__ void k_potts_transpose_out(const uint8_t* src, uint8_t* dst, int64_t n, int64_t n_chains, int64_t ld) {
    __shared__ uint8_t tile[32][33];
    const int64_t node0 = static_cast<int64_t>(blockIdx.x) * 32, chain0 = static_cast<int64_t>(blockIdx.y) * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int64_t node = node0 + r, chain = chain0 + threadIdx.x;
        tile[r][threadIdx.x] = (node < n && chain < n_chains) ? src[node * ld + chain] : 0;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int64_t chain = chain0 + r, node = node0 + threadIdx.x;
        if (chain < n_chains && node < n) dst[chain * n + node] = tile[threadIdx.x][r];
    }
}

int32_t palloc(DevBuf& b, size_t bytes) { return b.alloc(bytes); }

}  // namespace

struct thrml_potts {
    thrml_ctx* ctx = nullptr;
    int device = 0;
    int32_t nx = 0, ny = 0, nz = 0, K = 0;
    int64_t n = 0, n_chains = 0, chain_offset = 0, ld = 0, n_obs = 0;
    DevBuf state, tables, pair_tables, unary, counts, scratch, n_obs_dev;
    float table_mag = 0.0f;
    int32_t noise = THRML_POTTS_NOISE_QUAD;
    bool pair = false;  // pre-added direction tables exist (category counts with a compile-time kernel and 3 K^3 floats of shared memory to spare)
};

extern "C" {

int32_t thrml_potts_create(thrml_ctx* ctx, int32_t nx, int32_t ny, int32_t nz, int32_t n_categories, const float* tables, const float* unary, float beta,
                           int64_t n_chains, int64_t chain_offset, thrml_potts** out) {
    if (!ctx || !out || !tables) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (nx < 2 || ny < 2 || nz < 2 || (nx & 1) || (ny & 1) || (nz & 1)) return fail(THRML_ERR_INVALID_ARG, "lattice sides must be even and at least 2 (a two-colouring of the torus needs even sides)");
    if (n_categories < 1 || n_categories > MAX_K) return fail(THRML_ERR_INVALID_ARG, "n_categories must be between 1 and 32");
    if (n_chains < 1 || chain_offset < 0 || (chain_offset & 15)) return fail(THRML_ERR_INVALID_ARG, "n_chains must be positive and chain_offset a non-negative multiple of 16");
    const int64_t n = static_cast<int64_t>(nx) * ny * nz;
    if (n / 2 > (int64_t(1) << 32)) return fail(THRML_ERR_UNSUPPORTED, "more than 2^32 nodes per colour");
    CU_TRY(cudaSetDevice(ctx->device));
    auto P = std::make_unique<thrml_potts>();
    P->ctx = ctx; P->device = ctx->device;
    P->nx = nx; P->ny = ny; P->nz = nz; P->K = n_categories; P->n = n;
    P->n_chains = n_chains; P->chain_offset = chain_offset; P->ld = (n_chains + 15) / 16 * 16;
    const int K = n_categories;
    std::vector<float> tab(static_cast<size_t>(3) * K * K), un(static_cast<size_t>(n) * K, 0.0f);
    for (size_t i = 0; i < tab.size(); ++i) tab[i] = beta * tables[i];
    if (unary) for (size_t i = 0; i < un.size(); ++i) un[i] = beta * unary[i];
    if (int32_t rc = palloc(P->state, static_cast<size_t>(n) * P->ld)) return rc;
    if (int32_t rc = palloc(P->tables, tab.size() * 4)) return rc;
    if (int32_t rc = palloc(P->unary, un.size() * 4)) return rc;
    std::vector<float> pair;
    for (int d = 0; d < 3; ++d) {
        float m = 0.0f;
        for (int i = 0; i < K * K; ++i) m = std::max(m, std::fabs(tab[static_cast<size_t>(d) * K * K + i]));
        P->table_mag += 2.0f * m;
    }
    P->pair = (K == 3 || K == 4 || K == 5 || K == 8 || K == 10) && std::isfinite(P->table_mag);
    if (P->pair) {
        pair.resize(static_cast<size_t>(3) * K * K * K);
        for (int d = 0; d < 3; ++d)
            for (int c = 0; c < K; ++c)
                for (int sp = 0; sp < K; ++sp)
                    for (int sm = 0; sm < K; ++sm)
                        pair[((static_cast<size_t>(d) * K + c) * K + sp) * K + sm] =
                            static_cast<float>(static_cast<double>(tab[(static_cast<size_t>(d) * K + c) * K + sp]) + static_cast<double>(tab[(static_cast<size_t>(d) * K + sm) * K + c]));
        if (int32_t rc = palloc(P->pair_tables, pair.size() * 4)) return rc;
    }
    if (int32_t rc = palloc(P->counts, static_cast<size_t>(n) * K * 4)) return rc;
    cudaStream_t st = ctx->stream;
    CU_TRY(cudaMemsetAsync(P->state.p, 0, P->state.bytes, st));
    CU_TRY(cudaMemsetAsync(P->counts.p, 0, P->counts.bytes, st));
    CU_TRY(cudaMemcpyAsync(P->tables.p, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, st));
    CU_TRY(cudaMemcpyAsync(P->unary.p, un.data(), un.size() * 4, cudaMemcpyHostToDevice, st));
    if (P->pair) CU_TRY(cudaMemcpyAsync(P->pair_tables.p, pair.data(), pair.size() * 4, cudaMemcpyHostToDevice, st));
    CU_TRY(cudaStreamSynchronize(st));
    *out = P.release();
    return THRML_OK;
}
void thrml_potts_destroy(thrml_potts* P) {
    if (!P) return;
    cudaSetDevice(P->device);
    cudaDeviceSynchronize();
    delete P;
}
int32_t thrml_potts_set_noise(thrml_potts* P, int32_t mapping) {
    if (!P) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    if (mapping != THRML_POTTS_NOISE_PROGRAM && mapping != THRML_POTTS_NOISE_QUAD) return fail(THRML_ERR_INVALID_ARG, "unknown noise mapping");
    P->noise = mapping;
    return THRML_OK;
}
static dim3 potts_grid(const thrml_potts* P) { return dim3(static_cast<unsigned>((P->n / 2 + 7) / 8), static_cast<unsigned>((P->ld / 4 + 31) / 32)); }

int32_t thrml_potts_randomize(thrml_potts* P, uint64_t key) {
    if (!P) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    CU_TRY(cudaSetDevice(P->device));
    uint64_t keys[2];
    rng_split(key, 2, keys);
    for (int c = 0; c < 2; ++c) {
        k_potts_randomize<<<potts_grid(P), dim3(32, 8), 0, P->ctx->stream>>>(static_cast<uint8_t*>(P->state.p), P->nx, P->ny, P->nz, P->K, c, P->ld, P->n_chains,
                                                                            static_cast<uint32_t>(P->chain_offset >> 2), static_cast<uint32_t>(keys[c]), static_cast<uint32_t>(keys[c] >> 32));
        CU_TRY(cudaGetLastError());
    }
    return THRML_OK;
}
// The update kernel can count the categories it draws (the marginal observation that follows a sweep) when a warp's 32 lanes
// all hold chains of the state and the categories fit the 8-bit count fields.
static bool potts_counts_ride_along(const thrml_potts* P) { return P->K <= 16 && P->ld % 128 == 0 && P->ld <= 63 * 128; }
// Update one colour with its block key (asynchronous); `count`: add the draws to the category counts.
static int32_t potts_update(thrml_potts* P, int32_t colour, uint64_t block_key, bool count) {
    if (!P || colour < 0 || colour > 1) return fail(THRML_ERR_INVALID_ARG, "bad colour");
    CU_TRY(cudaSetDevice(P->device));
    PottsArgs a{static_cast<uint8_t*>(P->state.p), static_cast<const float*>(P->tables.p), static_cast<const float*>(P->unary.p), P->nx, P->ny, P->nz, P->K, colour, P->ld, P->n_chains,
                static_cast<uint32_t>(P->chain_offset >> 2), static_cast<uint32_t>(block_key), static_cast<uint32_t>(block_key >> 32)};
    a.pair_tables = static_cast<const float*>(P->pair_tables.p);
    a.table_mag = P->table_mag;
    a.counts = count ? static_cast<int32_t*>(P->counts.p) : nullptr;
    // CTAs stride over the nodes: about four waves of resident CTAs (three per SM), so each stages the tables a few times at most
    dim3 grid(potts_grid(P).x, 1);
    const dim3 block(32, 8);
    grid.x = std::min(grid.x, static_cast<unsigned>(P->ctx->sm_count) * 3u * 4u);
    const size_t smem = static_cast<size_t>(3) * P->K * P->K * (P->pair ? 1 + P->K : 1) * 4;
    const bool quad = P->noise == THRML_POTTS_NOISE_QUAD;
#define POTTS_LAUNCH(KT, PAIR)                                                          \
    do {                                                                                \
        if (quad) k_potts_update<KT, PAIR, true><<<grid, block, smem, P->ctx->stream>>>(a);  \
        else k_potts_update<KT, PAIR, false><<<grid, block, smem, P->ctx->stream>>>(a);      \
    } while (0)
    switch (P->pair ? P->K : 0) {
        case 3: POTTS_LAUNCH(3, true); break;
        case 4: POTTS_LAUNCH(4, true); break;
        case 5: POTTS_LAUNCH(5, true); break;
        case 8: POTTS_LAUNCH(8, true); break;
        case 10: POTTS_LAUNCH(10, true); break;
        default: POTTS_LAUNCH(0, false); break;
    }
#undef POTTS_LAUNCH
    CU_TRY(cudaGetLastError());
    return THRML_OK;
}
int32_t thrml_potts_update(thrml_potts* P, int32_t colour, uint64_t block_key) { return potts_update(P, colour, block_key, false); }
int32_t thrml_potts_observe_marginals(thrml_potts* P) {
    if (!P) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    CU_TRY(cudaSetDevice(P->device));
    if (P->K <= 10 && P->n_chains <= 2016)
        k_potts_marginals_packed<<<static_cast<unsigned>((P->n + 15) / 16), dim3(32, 8), 0, P->ctx->stream>>>(static_cast<const uint8_t*>(P->state.p), P->n, P->K, P->ld,
                                                                                                           P->n_chains, static_cast<int32_t*>(P->counts.p));
    else
        k_potts_marginals<<<static_cast<unsigned>((P->n + 7) / 8), dim3(32, 8), 0, P->ctx->stream>>>(static_cast<const uint8_t*>(P->state.p), P->n, P->K, P->ld, P->n_chains,
                                                                                                    static_cast<int32_t*>(P->counts.p));
    CU_TRY(cudaGetLastError());
    P->n_obs += P->n_chains;
    return THRML_OK;
}
int32_t thrml_potts_reset_marginals(thrml_potts* P) {
    if (!P) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    CU_TRY(cudaSetDevice(P->device));
    CU_TRY(cudaMemsetAsync(P->counts.p, 0, P->counts.bytes, P->ctx->stream));
    P->n_obs = 0;
    return THRML_OK;
}
int32_t thrml_potts_read_marginals(thrml_potts* P, int32_t* counts_out, int64_t* n_obs_out) {
    if (!P) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    CU_TRY(cudaSetDevice(P->device));
    if (counts_out) CU_TRY(cudaMemcpyAsync(counts_out, P->counts.p, P->counts.bytes, cudaMemcpyDeviceToHost, P->ctx->stream));
    CU_TRY(cudaStreamSynchronize(P->ctx->stream));
    if (n_obs_out) *n_obs_out = P->n_obs;
    return THRML_OK;
}
// run_blocks (sampling.rs:81-106): keys = key.split(n_iters); each sweep (sample_blocks, sampling.rs:28-63) splits its key
// in two block keys, colour 0 then colour 1.  Asynchronous.
// `observe`: the marginal observation that follows the last sweep (fused into that sweep's updates when they can count).
static int32_t potts_run(thrml_potts* P, uint64_t key, int64_t n_iters, bool observe) {
    if (!P) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    if (n_iters < 0) return fail(THRML_ERR_INVALID_ARG, "n_iters must be non-negative");
    std::vector<uint64_t> keys(static_cast<size_t>(n_iters));
    rng_split(key, n_iters, keys.data());
    const bool ride = observe && n_iters > 0 && potts_counts_ride_along(P);
    for (int64_t it = 0; it < n_iters; ++it) {
        uint64_t k2[2];
        rng_split(keys[it], 2, k2);
        for (int colour = 0; colour < 2; ++colour)
            if (int32_t rc = potts_update(P, colour, k2[colour], ride && it + 1 == n_iters)) return rc;
    }
    if (ride) P->n_obs += P->n_chains;
    else if (observe) return thrml_potts_observe_marginals(P);
    return THRML_OK;
}
int32_t thrml_potts_run_blocks(thrml_potts* P, uint64_t key, int64_t n_iters) { return potts_run(P, key, n_iters, false); }
// sample_with_observation (sampling.rs:178-320) with the category-marginal observer: key.split_two -> warm-up, observe,
// then n_samples - 1 times (steps_per_sample sweeps, observe); nothing after the first observation when n_samples <= 1.
int32_t thrml_potts_sample_with_marginals(thrml_potts* P, uint64_t key, int64_t n_warmup, int64_t n_samples, int64_t steps_per_sample) {
    if (!P) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    if (n_warmup < 0 || n_samples < 0 || steps_per_sample < 0) return fail(THRML_ERR_INVALID_ARG, "schedule entries must be non-negative");
    uint64_t two[2];
    rng_split(key, 2, two);
    if (int32_t rc = potts_run(P, two[0], n_warmup, true)) return rc;
    if (n_samples > 1) {
        std::vector<uint64_t> keys(static_cast<size_t>(n_samples - 1));
        rng_split(two[1], n_samples - 1, keys.data());
        for (int64_t i = 0; i < n_samples - 1; ++i)
            if (int32_t rc = potts_run(P, keys[i], steps_per_sample, true)) return rc;
    }
    CU_TRY(cudaStreamSynchronize(P->ctx->stream));
    return THRML_OK;
}
// Chains sharded over the ranks of `comm`: one ncclAllReduce adds the category counts (int32) in place on every rank; the
// observation counts are added alongside.
int32_t thrml_potts_marginals_allreduce(thrml_potts* P, thrml_comm* comm) {
    if (!P || !comm) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (comm->ctx != P->ctx) return fail(THRML_ERR_INVALID_ARG, "communicator and lattice belong to different contexts");
    if (comm->world == 1) return THRML_OK;
    const NcclApi* api = nccl_api();
    if (!api) return THRML_ERR_NCCL;
    CU_TRY(cudaSetDevice(P->device));
    cudaStream_t st = P->ctx->stream;
    if (int32_t rc = P->n_obs_dev.reserve(8)) return rc;
    const long long mine = P->n_obs;
    CU_TRY(cudaMemcpyAsync(P->n_obs_dev.p, &mine, 8, cudaMemcpyHostToDevice, st));
    NCCL_TRY(api, GroupStart());
    NCCL_TRY(api, AllReduce(P->n_obs_dev.p, P->n_obs_dev.p, 1, ncclInt64, ncclSum, comm->nccl, st));
    NCCL_TRY(api, AllReduce(P->counts.p, P->counts.p, static_cast<size_t>(P->n) * P->K, ncclInt32, ncclSum, comm->nccl, st));
    NCCL_TRY(api, GroupEnd());
    long long total = 0;
    CU_TRY(cudaMemcpyAsync(&total, P->n_obs_dev.p, 8, cudaMemcpyDeviceToHost, st));
    CU_TRY(cudaStreamSynchronize(st));
    P->n_obs = total;
    return THRML_OK;
}
static int32_t potts_scratch(thrml_potts* P, size_t bytes) {
    if (P->scratch.holds(bytes)) return THRML_OK;
    CU_TRY(cudaStreamSynchronize(P->ctx->stream));
    return palloc(P->scratch, bytes);
}
// State as category bytes, host layout [chain][node].
int32_t thrml_potts_upload(thrml_potts* P, const uint8_t* host) {
    if (!P || !host) return fail(THRML_ERR_INVALID_ARG, "null argument");
    CU_TRY(cudaSetDevice(P->device));
    const size_t bytes = static_cast<size_t>(P->n) * P->n_chains;
    if (int32_t rc = potts_scratch(P, bytes)) return rc;
    CU_TRY(cudaMemcpyAsync(P->scratch.p, host, bytes, cudaMemcpyHostToDevice, P->ctx->stream));
    dim3 grid(static_cast<unsigned>((P->n + 31) / 32), static_cast<unsigned>((P->ld + 31) / 32));
    k_potts_transpose_in<<<grid, dim3(32, 8), 0, P->ctx->stream>>>(static_cast<const uint8_t*>(P->scratch.p), static_cast<uint8_t*>(P->state.p), P->n, P->n_chains, P->ld);
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaStreamSynchronize(P->ctx->stream));
    return THRML_OK;
}
int32_t thrml_potts_download(thrml_potts* P, uint8_t* host) {
    if (!P || !host) return fail(THRML_ERR_INVALID_ARG, "null argument");
    CU_TRY(cudaSetDevice(P->device));
    const size_t bytes = static_cast<size_t>(P->n) * P->n_chains;
    if (int32_t rc = potts_scratch(P, bytes)) return rc;
    dim3 grid(static_cast<unsigned>((P->n + 31) / 32), static_cast<unsigned>((P->n_chains + 31) / 32));
    k_potts_transpose_out<<<grid, dim3(32, 8), 0, P->ctx->stream>>>(static_cast<const uint8_t*>(P->state.p), static_cast<uint8_t*>(P->scratch.p), P->n, P->n_chains, P->ld);
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaMemcpyAsync(host, P->scratch.p, bytes, cudaMemcpyDeviceToHost, P->ctx->stream));
    CU_TRY(cudaStreamSynchronize(P->ctx->stream));
    return THRML_OK;
}
int32_t thrml_potts_synchronize(thrml_potts* P) {
    if (!P) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    CU_TRY(cudaSetDevice(P->device));
    CU_TRY(cudaStreamSynchronize(P->ctx->stream));
    return THRML_OK;
}

}  // extern "C"
