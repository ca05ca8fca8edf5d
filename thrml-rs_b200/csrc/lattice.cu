// Implicit 2-D periodic Ising lattice with bit-packed state, for lattices too large for per-node tables
// (32768 x 32768 spins and beyond), sharded by row stripes.
//
// Semantics = IsingSamplingProgram (crates/thrml-models/src/ising.rs:342-388) on the nearest-neighbour torus of
// make_nearest_neighbor_lattice (crates/thrml-models/src/graph_utils.rs:177-243) with one coupling J, one bias b and the two
// checkerboard blocks [(row+col) even, (row+col) odd]; the field of a spin is accumulated in the reference's slot order
// (edges where the node is the smaller endpoint first, then those where it is the larger, each in (min,max) edge order)
// so the sampled states equal those of the explicit program bit for bit.  That order differs at the lattice seams, hence
// one 16-entry threshold table per seam class.
//
// Layout: plane[colour][stripe row + 1][word][chain] u32, 32 spins of one colour and one row per word, chains innermost;
// stripe rows 0 and n_rows+1 are halo rows holding the neighbouring stripes' boundary rows.
#include <algorithm>
#include <cstring>
#include <memory>
#include <vector>

#include "comm.h"
#include "ctx.h"
#include "devbuf.h"
#include "device_math.cuh"

using namespace thrml;

namespace {

// neighbour bit positions inside a 4-bit configuration
constexpr int NB_UP = 0, NB_LEFT = 1, NB_RIGHT = 2, NB_DOWN = 3;

struct LatArgs {
    uint32_t* own;          // plane of the colour being updated (with halo rows)
    const uint32_t* other;  // plane of the other colour
    const uint32_t* lut;    // [9][16] thresholds
    int64_t H, W;           // whole lattice
    int64_t row0;           // first global row of the stripe
    int32_t n_rows, words, chains, colour;
    uint32_t chain_word0;
    PhiloxRoundKeys rk;  // round keys of the block key, computed once on the host
    uint32_t vmask[8][5];  // bit-sliced mapping: all-ones where bit b of the threshold's top byte is set for s up neighbours
    long long* record;     // [2][chains] sums to add this pass's observables to, or null
};

// One thread = one word (32 spins of one row and colour) x four chains.  The four neighbour bits of each spin are
// gathered eight spins at a time: a 256-entry shared table spreads a byte of a neighbour word to one bit per nibble, the
// four spread words are combined with multiply-adds, and each nibble then indexes the threshold table directly.
__global__ void __launch_bounds__(128) k_lattice_update(const __grid_constant__ LatArgs a, int32_t row_begin, int32_t row_end) {
    __shared__ uint32_t s_lut[9 * 16];
    __shared__ uint32_t s_spread[256];
    for (int i = threadIdx.x; i < 9 * 16; i += blockDim.x) s_lut[i] = a.lut[i];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
        uint32_t v = 0;
#pragma unroll
        for (int bit = 0; bit < 8; ++bit) v |= ((static_cast<uint32_t>(i) >> bit) & 1u) << (4 * bit);
        s_spread[i] = v;
    }
    __syncthreads();
    const int quads = a.chains >> 2;
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t per_row = static_cast<int64_t>(a.words) * quads;
    const int64_t total = static_cast<int64_t>(row_end - row_begin) * per_row;
    if (gid >= total) return;
    const int r = row_begin + static_cast<int>(gid / per_row);  // stripe row 0..n_rows-1
    const int w = static_cast<int>((gid % per_row) / quads);
    const int q = static_cast<int>(gid % quads);
    const int64_t gi = a.row0 + r;                               // global row
    const int p = static_cast<int>((gi + a.colour) & 1);         // column parity of this colour in this row: col = 2*jj + p
    auto at = [&](const uint32_t* plane, int srow, int word) {
        return *reinterpret_cast<const uint4*>(plane + (static_cast<int64_t>(srow) * a.words + word) * a.chains + 4 * q);
    };
    const uint4 up = at(a.other, r, w), down = at(a.other, r + 2, w), same = at(a.other, r + 1, w);
    const int wadj = p == 0 ? (w == 0 ? a.words - 1 : w - 1) : (w == a.words - 1 ? 0 : w + 1);
    const uint4 adj = at(a.other, r + 1, wadj);
    // p == 0: left neighbour is jj-1 (shifted in from the previous word), right neighbour is jj; p == 1: left is jj, right is jj+1
    uint32_t U[4] = {up.x, up.y, up.z, up.w}, D[4] = {down.x, down.y, down.z, down.w}, L[4], R[4];
    const uint32_t S[4] = {same.x, same.y, same.z, same.w}, A[4] = {adj.x, adj.y, adj.z, adj.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        if (p == 0) { L[c] = (S[c] << 1) | (A[c] >> 31); R[c] = S[c]; }
        else { L[c] = S[c]; R[c] = (S[c] >> 1) | (A[c] << 31); }
    }
    const int row_cls = gi == 0 ? 1 : (gi == a.H - 1 ? 2 : 0);
    const bool first_col = p == 0 && w == 0, last_col = p == 1 && w == a.words - 1;
    const uint32_t node_base = static_cast<uint32_t>(gi * (a.W >> 1) + 32 * static_cast<int64_t>(w));
    uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll 1
    for (int g = 0; g < 4; ++g) {
        // nibble j of P[c] = configuration (up | left<<1 | right<<2 | down<<3) of spin 8g+j of chain c
        uint32_t P[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t su = s_spread[(U[c] >> (8 * g)) & 0xffu], sl = s_spread[(L[c] >> (8 * g)) & 0xffu];
            const uint32_t sr = s_spread[(R[c] >> (8 * g)) & 0xffu], sd = s_spread[(D[c] >> (8 * g)) & 0xffu];
            P[c] = su + 2u * sl + 4u * sr + 8u * sd;
        }
        uint32_t byte[4] = {0, 0, 0, 0};  // the eight new spins of this group, per chain: constant bit positions inside the group
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int k = 8 * g + j;
            const U4 rr = philox4x32_10_rk(node_base + k, a.chain_word0 + q, 0u, TAG_SPIN, a.rk);
            const uint32_t rnd[4] = {rr.x, rr.y, rr.z, rr.w};
            int col_cls = 0;
            if (j == 0) col_cls = (g == 0 && first_col) ? 1 : 0;
            if (j == 7) col_cls = (g == 3 && last_col) ? 2 : 0;
            const uint32_t* T = s_lut + (row_cls * 3 + col_cls) * 16;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t cfg = (P[c] >> (4 * j)) & 15u;
                byte[c] |= rnd[c] <= T[cfg] ? (1u << j) : 0u;
            }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) out[c] |= byte[c] << (8 * g);
    }
    *reinterpret_cast<uint4*>(a.own + (static_cast<int64_t>(r + 1) * a.words + w) * a.chains + 4 * q) = make_uint4(out[0], out[1], out[2], out[3]);
}

// The update with the engine's bit-sliced noise mapping (thrml_lattice_set_noise, mapping 1).  The 32-bit word a spin's draw
// compares with its threshold is assembled from counter-based calls that are shared as widely as the layout allows:
//     top byte, bit b  = bit (n & 31) of word (b & 3) of Philox(n >> 5, chain, 1 + (b >> 2), TAG_SPIN)   -- two calls serve 32 spins
//     low 24 bits      = low 24 bits of word (chain & 3) of Philox(n, chain >> 2, 3, TAG_SPIN)
// (n = index of the spin inside its colour block, chain = global chain id).  The top byte alone decides unless it equals
// the threshold's top byte (one draw in 256); only then is the third call made.  Same rule `word <= threshold`, same
// 24-bit resolution of the uniform.
// The top bytes of 32 spins arrive as eight bit planes, so the comparison runs bit-sliced on whole words: the four neighbour
// words are added into three sum planes, the threshold's top byte — when it depends on the configuration only through the
// number of up neighbours (SYM, checked on the host for every seam class) — becomes eight planes of a five-way select, and
// a ripple comparator from the low bit up yields `less` and `equal` for 32 spins in two logic operations per bit.  Without
// that symmetry the same mapping is evaluated spin by spin from the threshold table.
// RECORD (the second colour of a sweep): every bond joins the two colours, so this pass sees each bond once and each word
// of the other colour once; per chain it adds the sum of spins and the sum of bond products to `record`.
// CTAs stride over the words; a thread keeps its chain quad for the whole launch.
template <bool SYM, bool RECORD>
__global__ void __launch_bounds__(128, 4) k_lattice_update_sliced(const __grid_constant__ LatArgs a, int32_t row_begin, int32_t row_end) {
    __shared__ uint32_t s_lut[9 * 16];
    for (int i = threadIdx.x; i < 9 * 16; i += blockDim.x) s_lut[i] = a.lut[i];
    __syncthreads();
    const int quads = a.chains >> 2;
    const int64_t per_row = static_cast<int64_t>(a.words) * quads;
    const int64_t total = static_cast<int64_t>(row_end - row_begin) * per_row;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;  // a multiple of 128, hence of `quads`
    int32_t spins[4] = {0, 0, 0, 0}, agree[4] = {0, 0, 0, 0};
    const int q = static_cast<int>((static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) % quads);
    // (row, word) of this thread's items advance by a fixed amount per iteration: no division inside the loop
    const int64_t gid0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int step_rows = static_cast<int>(step / per_row), step_words = static_cast<int>((step % per_row) / quads);
    int r = row_begin + static_cast<int>(gid0 / per_row), w = static_cast<int>((gid0 % per_row) / quads);
    for (int64_t gid = gid0; gid < total; gid += step, r += step_rows, w += step_words) {
        if (w >= a.words) {
            w -= a.words;
            ++r;
        }
        const int64_t gi = a.row0 + r;
        const int p = static_cast<int>((gi + a.colour) & 1);
        auto at = [&](const uint32_t* plane, int srow, int word) {
            return *reinterpret_cast<const uint4*>(plane + (static_cast<int64_t>(srow) * a.words + word) * a.chains + 4 * q);
        };
        const uint4 up = at(a.other, r, w), down = at(a.other, r + 2, w), same = at(a.other, r + 1, w);
        const int wadj = p == 0 ? (w == 0 ? a.words - 1 : w - 1) : (w == a.words - 1 ? 0 : w + 1);
        const uint4 adj = at(a.other, r + 1, wadj);
        const uint32_t U[4] = {up.x, up.y, up.z, up.w}, D[4] = {down.x, down.y, down.z, down.w};
        const uint32_t S[4] = {same.x, same.y, same.z, same.w}, A[4] = {adj.x, adj.y, adj.z, adj.w};
        const int row_cls = gi == 0 ? 1 : (gi == a.H - 1 ? 2 : 0);
        const bool first_col = p == 0 && w == 0, last_col = p == 1 && w == a.words - 1;
        const uint32_t node_base = static_cast<uint32_t>(gi * (a.W >> 1) + 32 * static_cast<int64_t>(w));  // a multiple of 32
        uint32_t out[4], tie[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t Lc = p == 0 ? ((S[c] << 1) | (A[c] >> 31)) : S[c], Rc = p == 0 ? S[c] : ((S[c] >> 1) | (A[c] << 31));
            const uint32_t chain = 4u * (a.chain_word0 + static_cast<uint32_t>(q)) + c;
            const U4 ra = philox4x32_10_rk(node_base >> 5, chain, 1u, TAG_SPIN, a.rk), rb = philox4x32_10_rk(node_base >> 5, chain, 2u, TAG_SPIN, a.rk);
            const uint32_t rnd[8] = {ra.x, ra.y, ra.z, ra.w, rb.x, rb.y, rb.z, rb.w};  // plane b: bit k = bit b of spin k's top byte
            uint32_t lt = 0u, eq = 0xffffffffu;
            if (SYM) {
                // number of up neighbours per spin as three planes (0..4)
                const uint32_t x0 = U[c] ^ Lc, x1 = U[c] & Lc, y0 = Rc ^ D[c], y1 = Rc & D[c];
                const uint32_t s0 = x0 ^ y0, c0 = x0 & y0, s1 = x1 ^ y1 ^ c0, s2 = x1 & y1;
#pragma unroll
                for (int b = 0; b < 8; ++b) {
                    const uint32_t lo = (s0 & a.vmask[b][1]) | (~s0 & a.vmask[b][0]), hi = (s0 & a.vmask[b][3]) | (~s0 & a.vmask[b][2]);
                    const uint32_t mid = (s1 & hi) | (~s1 & lo);
                    const uint32_t t = (s2 & a.vmask[b][4]) | (~s2 & mid);  // bit b of the threshold's top byte, per spin
                    const uint32_t x = rnd[b] ^ t;
                    lt = (t & ~rnd[b]) | (~x & lt);  // less so far, from the low bit up: a higher bit overrides
                    eq &= ~x;
                }
            } else {
                lt = 0u;
                eq = 0u;
#pragma unroll 1
                for (int k = 0; k < 32; ++k) {
                    uint32_t h8 = 0;
#pragma unroll
                    for (int b = 0; b < 8; ++b) h8 |= ((rnd[b] >> k) & 1u) << b;
                    const uint32_t cfg = ((U[c] >> k) & 1u) | (((Lc >> k) & 1u) << 1) | (((Rc >> k) & 1u) << 2) | (((D[c] >> k) & 1u) << 3);
                    const int col_cls = (k == 0 && first_col) ? 1 : ((k == 31 && last_col) ? 2 : 0);
                    const uint32_t T8 = s_lut[(row_cls * 3 + col_cls) * 16 + cfg] >> 24;
                    lt |= (h8 < T8 ? 1u : 0u) << k;
                    eq |= (h8 == T8 ? 1u : 0u) << k;
                }
            }
            out[c] = lt;
            tie[c] = eq;
        }
        // Ties (top bytes equal, one draw in 256): the low 24 bits of the draw decide.  They come from a call keyed by the spin
        // whose four words serve the four chains, so the chains' ties are resolved together, one call per tied spin position:
        // a warp runs this loop as often as its busiest lane has tied positions, once for the four chains instead of once each.
        for (uint32_t m = tie[0] | tie[1] | tie[2] | tie[3]; m; m &= m - 1u) {
            const int k = __ffs(m) - 1;
            const U4 rr = philox4x32_10_rk(node_base + k, a.chain_word0 + q, 3u, TAG_SPIN, a.rk);
            const int col_cls = (k == 0 && first_col) ? 1 : ((k == 31 && last_col) ? 2 : 0);
            const uint32_t* tab = s_lut + (row_cls * 3 + col_cls) * 16;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (!((tie[c] >> k) & 1u)) continue;
                const uint32_t Lc = p == 0 ? ((S[c] << 1) | (A[c] >> 31)) : S[c], Rc = p == 0 ? S[c] : ((S[c] >> 1) | (A[c] << 31));
                const uint32_t cfg = ((U[c] >> k) & 1u) | (((Lc >> k) & 1u) << 1) | (((Rc >> k) & 1u) << 2) | (((D[c] >> k) & 1u) << 3);
                out[c] |= ((pick(rr, c) & 0xffffffu) <= (tab[cfg] & 0xffffffu) ? 1u : 0u) << k;
            }
        }
        if (RECORD) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t Lc = p == 0 ? ((S[c] << 1) | (A[c] >> 31)) : S[c], Rc = p == 0 ? S[c] : ((S[c] >> 1) | (A[c] << 31));
                spins[c] += __popc(out[c]) + __popc(S[c]);
                agree[c] += __popc(~(out[c] ^ U[c])) + __popc(~(out[c] ^ D[c])) + __popc(~(out[c] ^ Lc)) + __popc(~(out[c] ^ Rc));
            }
        }
        *reinterpret_cast<uint4*>(a.own + (static_cast<int64_t>(r + 1) * a.words + w) * a.chains + 4 * q) = make_uint4(out[0], out[1], out[2], out[3]);
    }
    if (RECORD) {
        // words seen by this thread: every one holds 32 spins of each colour and 128 bonds
        int64_t items = 0;
        {
            const int64_t first = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
            if (first < total) items = (total - first + step - 1) / step;
        }
        const int lane = threadIdx.x & 31;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            long long sp = 2LL * spins[c] - 64LL * items, bo = 2LL * agree[c] - 128LL * items;
            for (int off = 16; off >= quads && off >= 1; off >>= 1) {  // lanes that share the chain quad
                sp += __shfl_xor_sync(0xffffffffu, sp, off);
                bo += __shfl_xor_sync(0xffffffffu, bo, off);
            }
            if (lane < quads || quads > 32) {
                atomicAdd(reinterpret_cast<unsigned long long*>(a.record + 4 * q + c), static_cast<unsigned long long>(sp));
                atomicAdd(reinterpret_cast<unsigned long long*>(a.record + a.chains + 4 * q + c), static_cast<unsigned long long>(bo));
            }
        }
    }
}

// Threshold tables: gamma = (0 + b) + (((0 + t1) + t2) + t3) + t4 with the neighbours taken in `order`, exactly as the
// explicit program accumulates them; threshold as in the table kernel of the explicit engine.
__global__ void k_lattice_build_lut(float J, float b, const int32_t* order /*[9][4]*/, uint32_t* lut) {
    const int cls = threadIdx.x >> 4, cfg = threadIdx.x & 15;
    if (cls >= 9) return;
    float gs = 0.0f;
    for (int s = 0; s < 4; ++s) {
        const int bit = order[cls * 4 + s];
        gs = __fadd_rn(gs, __fmul_rn(J, ((cfg >> bit) & 1) ? 1.0f : -1.0f));
    }
    const float gamma = __fadd_rn(__fadd_rn(0.0f, b), gs);
    const float pr = det_sigmoid(__fmul_rn(gamma, 2.0f));
    const uint32_t fl = static_cast<uint32_t>(__fmul_rn(pr, 16777216.0f));
    lut[threadIdx.x] = fl >= 16777216u ? 0xffffffffu : ((fl << 8) | 0xffu);
}

// Uniform random start, same stream as thrml_state_randomize on the explicit program (spin = top bit of the word).
__global__ void __launch_bounds__(128) k_lattice_randomize(uint32_t* plane, int64_t W, int64_t row0, int32_t n_rows, int32_t words, int32_t chains,
                                                          uint32_t chain_word0, uint32_t k0, uint32_t k1) {
    const int quads = chains >> 2;
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t per_row = static_cast<int64_t>(words) * quads;
    if (gid >= static_cast<int64_t>(n_rows) * per_row) return;
    const int r = static_cast<int>(gid / per_row), w = static_cast<int>((gid % per_row) / quads), q = static_cast<int>(gid % quads);
    const uint32_t node_base = static_cast<uint32_t>((row0 + r) * (W >> 1) + 32 * static_cast<int64_t>(w));
    uint32_t out[4] = {0, 0, 0, 0};
    for (int k = 0; k < 32; ++k) {
        const U4 rr = philox4x32_10(node_base + k, chain_word0 + q, 0u, TAG_RAND, k0, k1);
        out[0] |= (rr.x >> 31) << k;
        out[1] |= (rr.y >> 31) << k;
        out[2] |= (rr.z >> 31) << k;
        out[3] |= (rr.w >> 31) << k;
    }
    *reinterpret_cast<uint4*>(plane + (static_cast<int64_t>(r + 1) * words + w) * chains + 4 * q) = make_uint4(out[0], out[1], out[2], out[3]);
}

// Per chain: sum of spins (both colours) and sum over bonds of s_i s_j, each bond counted from its colour-0 end.
__global__ void __launch_bounds__(256) k_lattice_observe(const uint32_t* p0, const uint32_t* p1, int64_t row0, int32_t n_rows, int32_t words, int32_t chains,
                                                        long long* out /*[2][chains]*/) {
    const int chain = threadIdx.x % chains;  // blockDim.x is a multiple of chains
    const int lanes_per_chain = blockDim.x / chains;
    const int64_t cells = static_cast<int64_t>(n_rows) * words;
    long long spins = 0, bonds = 0;
    for (int64_t cell = static_cast<int64_t>(blockIdx.x) * lanes_per_chain + threadIdx.x / chains; cell < cells; cell += static_cast<int64_t>(gridDim.x) * lanes_per_chain) {
        const int r = static_cast<int>(cell / words), w = static_cast<int>(cell % words);
        const int p = static_cast<int>((row0 + r) & 1);  // colour 0: col = 2*jj + p
        auto at = [&](const uint32_t* plane, int srow, int word) { return plane[(static_cast<int64_t>(srow) * words + word) * chains + chain]; };
        const uint32_t s0 = at(p0, r + 1, w), s1 = at(p1, r + 1, w);
        spins += 2 * (__popc(s0) + __popc(s1)) - 64;
        const int wadj = p == 0 ? (w == 0 ? words - 1 : w - 1) : (w == words - 1 ? 0 : w + 1);
        const uint32_t adj = at(p1, r + 1, wadj);
        const uint32_t left = p == 0 ? ((s1 << 1) | (adj >> 31)) : s1, right = p == 0 ? s1 : ((s1 >> 1) | (adj << 31));
        const int agree = __popc(~(s0 ^ at(p1, r, w))) + __popc(~(s0 ^ at(p1, r + 2, w))) + __popc(~(s0 ^ left)) + __popc(~(s0 ^ right));
        bonds += 2 * agree - 128;
    }
    atomicAdd(reinterpret_cast<unsigned long long*>(out + chain), static_cast<unsigned long long>(spins));
    atomicAdd(reinterpret_cast<unsigned long long*>(out + chains + chain), static_cast<unsigned long long>(bonds));
}

// host layout [chain][row][col] bytes (0/1) <-> bit planes, one thread per (row, word, chain)
__global__ void k_lattice_pack(const uint8_t* host_order, uint32_t* p0, uint32_t* p1, int64_t W, int64_t row0, int32_t n_rows, int32_t words, int32_t chains) {
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= static_cast<int64_t>(n_rows) * words * chains) return;
    const int chain = static_cast<int>(gid % chains), w = static_cast<int>((gid / chains) % words), r = static_cast<int>(gid / (static_cast<int64_t>(chains) * words));
    const uint8_t* src = host_order + (static_cast<int64_t>(chain) * n_rows + r) * W;
    for (int colour = 0; colour < 2; ++colour) {
        const int p = static_cast<int>((row0 + r + colour) & 1);
        uint32_t word = 0;
        for (int k = 0; k < 32; ++k) word |= static_cast<uint32_t>(src[2 * (32 * w + k) + p] & 1u) << k;
        (colour ? p1 : p0)[(static_cast<int64_t>(r + 1) * words + w) * chains + chain] = word;
    }
}
__global__ void k_lattice_unpack(const uint32_t* p0, const uint32_t* p1, uint8_t* host_order, int64_t W, int64_t row0, int32_t n_rows, int32_t words, int32_t chains) {
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= static_cast<int64_t>(n_rows) * words * chains) return;
    const int chain = static_cast<int>(gid % chains), w = static_cast<int>((gid / chains) % words), r = static_cast<int>(gid / (static_cast<int64_t>(chains) * words));
    uint8_t* dst = host_order + (static_cast<int64_t>(chain) * n_rows + r) * W;
    for (int colour = 0; colour < 2; ++colour) {
        const int p = static_cast<int>((row0 + r + colour) & 1);
        const uint32_t word = (colour ? p1 : p0)[(static_cast<int64_t>(r + 1) * words + w) * chains + chain];
        for (int k = 0; k < 32; ++k) dst[2 * (32 * w + k) + p] = (word >> k) & 1u;
    }
}

}  // namespace

// Bit-packed host layout: bits[chain][stripe row][W / 32] u32, bit k of word v = column 32 v + k.  A plane word holds 32
// spins of one colour: columns 2 (32 w + k) + p, i.e. the bits of parity p of host words 2w and 2w + 1.
__device__ __forceinline__ uint32_t even_bits(uint32_t x) {  // bits 0, 2, 4, ... of x packed into the low 16 bits
    x &= 0x55555555u;
    x = (x | (x >> 1)) & 0x33333333u;
    x = (x | (x >> 2)) & 0x0f0f0f0fu;
    x = (x | (x >> 4)) & 0x00ff00ffu;
    x = (x | (x >> 8)) & 0x0000ffffu;
    return x;
}
__device__ __forceinline__ uint32_t spread_bits(uint32_t x) {  // the low 16 bits of x moved to bits 0, 2, 4, ...
    x &= 0x0000ffffu;
    x = (x | (x << 8)) & 0x00ff00ffu;
    x = (x | (x << 4)) & 0x0f0f0f0fu;
    x = (x | (x << 2)) & 0x33333333u;
    x = (x | (x << 1)) & 0x55555555u;
    return x;
}
__global__ void k_lattice_pack_bits(const uint32_t* host_order, uint32_t* p0, uint32_t* p1, int64_t row0, int32_t n_rows, int32_t words, int32_t chains) {
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= static_cast<int64_t>(n_rows) * words * chains) return;
    const int chain = static_cast<int>(gid % chains), w = static_cast<int>((gid / chains) % words), r = static_cast<int>(gid / (static_cast<int64_t>(chains) * words));
    const uint32_t* src = host_order + (static_cast<int64_t>(chain) * n_rows + r) * (2 * words) + 2 * w;
    const uint32_t a = src[0], b = src[1];
    const uint32_t even = even_bits(a) | (even_bits(b) << 16), odd = even_bits(a >> 1) | (even_bits(b >> 1) << 16);
    const int p = static_cast<int>((row0 + r) & 1);  // colour 0 sits on the columns of parity p in this row
    const int64_t at = (static_cast<int64_t>(r + 1) * words + w) * chains + chain;
    p0[at] = p ? odd : even;
    p1[at] = p ? even : odd;
}
__global__ void k_lattice_unpack_bits(const uint32_t* p0, const uint32_t* p1, uint32_t* host_order, int64_t row0, int32_t n_rows, int32_t words, int32_t chains) {
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= static_cast<int64_t>(n_rows) * words * chains) return;
    const int chain = static_cast<int>(gid % chains), w = static_cast<int>((gid / chains) % words), r = static_cast<int>(gid / (static_cast<int64_t>(chains) * words));
    const int64_t at = (static_cast<int64_t>(r + 1) * words + w) * chains + chain;
    const int p = static_cast<int>((row0 + r) & 1);
    const uint32_t even = p ? p1[at] : p0[at], odd = p ? p0[at] : p1[at];
    uint32_t* dst = host_order + (static_cast<int64_t>(chain) * n_rows + r) * (2 * words) + 2 * w;
    dst[0] = spread_bits(even) | (spread_bits(odd) << 1);
    dst[1] = spread_bits(even >> 16) | (spread_bits(odd >> 16) << 1);
}

struct thrml_lattice {
    thrml_ctx* ctx = nullptr;
    int device = 0;
    int64_t H = 0, W = 0, row0 = 0, n_rows = 0, n_chains = 0, chain_offset = 0;
    int32_t words = 0;
    DevBuf plane[2], lut, order, obs, scratch;
    size_t row_bytes = 0;  // one row of one colour
    float coupling = 0.f, bias = 0.f;
    int32_t noise = 1;  // THRML_LATTICE_NOISE_*
    bool force_table = false;   // THRML_LATTICE_NOISE_PACKED_TABLE: take the table route even when the bit-sliced one applies
    bool symmetric = false;     // the thresholds' top bytes depend on the configuration only through the number of up neighbours
    uint32_t vmask[8][5] = {};  // the planes of that dependence
    // sweep driver: halo exchange on a side stream, overlapped with the interior rows
    cudaStream_t side = nullptr;
    cudaEvent_t ev_edge = nullptr, ev_halo = nullptr;
    // per-sweep observable series: record t holds, per chain, this stripe's sum of spins and sum of bond products
    DevBuf series;
    int64_t series_len = 0, series_cap = 0;
    long long* record_into = nullptr;  // set by the sweep driver around the second colour's launches: the update records the observables itself
    uint32_t* p(int c) const { return static_cast<uint32_t*>(plane[c].p); }
    ~thrml_lattice() {
        if (ev_edge) cudaEventDestroy(ev_edge);
        if (ev_halo) cudaEventDestroy(ev_halo);
        if (side) cudaStreamDestroy(side);
    }
};

static int32_t lat_alloc(DevBuf& b, size_t bytes) { return b.alloc(bytes); }

extern "C" {

int32_t thrml_lattice_create(thrml_ctx* ctx, int64_t height, int64_t width, int64_t row_begin, int64_t n_rows, float coupling, float bias, float beta,
                             int64_t n_chains, int64_t chain_offset, thrml_lattice** out) {
    if (!ctx || !out) return fail(THRML_ERR_INVALID_ARG, "null argument");
    if (height < 4 || (height & 1) || width < 64 || (width & 63)) return fail(THRML_ERR_INVALID_ARG, "lattice height must be even and >= 4, width a multiple of 64");
    if (row_begin < 0 || n_rows < 1 || row_begin + n_rows > height) return fail(THRML_ERR_INVALID_ARG, "stripe rows out of range");
    if (n_rows < 2 && n_rows != height) return fail(THRML_ERR_INVALID_ARG, "a stripe needs at least two rows");
    if (n_chains < 4 || (n_chains & 3) || n_chains > 256 || (256 % n_chains) != 0) return fail(THRML_ERR_INVALID_ARG, "n_chains must be 4, 8, 16, 32, 64, 128 or 256");
    if (chain_offset < 0 || (chain_offset & 3)) return fail(THRML_ERR_INVALID_ARG, "chain_offset must be a non-negative multiple of 4");
    if (height * (width / 2) > (int64_t(1) << 32)) return fail(THRML_ERR_UNSUPPORTED, "more than 2^32 spins per colour");
    CU_TRY(cudaSetDevice(ctx->device));
    auto L = std::make_unique<thrml_lattice>();
    L->ctx = ctx;
    L->device = ctx->device;
    L->H = height; L->W = width; L->row0 = row_begin; L->n_rows = n_rows; L->n_chains = n_chains; L->chain_offset = chain_offset;
    L->coupling = coupling; L->bias = bias;
    L->words = static_cast<int32_t>(width / 64);
    L->row_bytes = static_cast<size_t>(L->words) * n_chains * 4;
    for (int c = 0; c < 2; ++c) {
        if (int32_t rc = lat_alloc(L->plane[c], L->row_bytes * (n_rows + 2))) return rc;
        CU_TRY(cudaMemsetAsync(L->plane[c].p, 0, L->plane[c].bytes, ctx->stream));
    }
    if (int32_t rc = lat_alloc(L->lut, 9 * 16 * 4)) return rc;
    if (int32_t rc = lat_alloc(L->order, 9 * 4 * 4)) return rc;
    if (int32_t rc = lat_alloc(L->obs, 2 * n_chains * 8)) return rc;
    // canonical slot order per seam class: partners with a larger node index first (ascending), then the smaller ones
    // (ascending) — the order in which BlockSamplingProgram::new lists a node's edge rows (program.rs:101-134).
    std::vector<int32_t> order(9 * 4);
    for (int rc = 0; rc < 3; ++rc)
        for (int cc = 0; cc < 3; ++cc) {
            const int64_t i = rc == 1 ? 0 : (rc == 2 ? height - 1 : 1), j = cc == 1 ? 0 : (cc == 2 ? width - 1 : 1);
            const int64_t idx = i * width + j;
            std::pair<int64_t, int> nb[4] = {{((i + height - 1) % height) * width + j, NB_UP}, {i * width + (j + width - 1) % width, NB_LEFT},
                                             {i * width + (j + 1) % width, NB_RIGHT}, {((i + 1) % height) * width + j, NB_DOWN}};
            std::sort(nb, nb + 4);
            int s = 0;
            for (auto& n : nb) if (n.first > idx) order[(rc * 3 + cc) * 4 + s++] = n.second;
            for (auto& n : nb) if (n.first < idx) order[(rc * 3 + cc) * 4 + s++] = n.second;
        }
    CU_TRY(cudaMemcpyAsync(L->order.p, order.data(), order.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
    k_lattice_build_lut<<<1, 9 * 16, 0, ctx->stream>>>(beta * coupling, beta * bias, static_cast<const int32_t*>(L->order.p), static_cast<uint32_t*>(L->lut.p));
    CU_TRY(cudaGetLastError());
    {
        uint32_t h_lut[9 * 16];
        CU_TRY(cudaMemcpyAsync(h_lut, L->lut.p, sizeof(h_lut), cudaMemcpyDeviceToHost, ctx->stream));
        CU_TRY(cudaStreamSynchronize(ctx->stream));
        uint32_t top[5];
        bool sym = true;
        for (int sdx = 0; sdx <= 4; ++sdx) top[sdx] = 0x100u;  // unset
        for (int cls = 0; cls < 9 && sym; ++cls)
            for (int cfg = 0; cfg < 16; ++cfg) {
                const int ups = __builtin_popcount(static_cast<unsigned>(cfg));
                const uint32_t t8 = h_lut[cls * 16 + cfg] >> 24;
                if (top[ups] == 0x100u) top[ups] = t8;
                else if (top[ups] != t8) { sym = false; break; }
            }
        L->symmetric = sym;
        if (sym)
            for (int b = 0; b < 8; ++b)
                for (int sdx = 0; sdx <= 4; ++sdx) L->vmask[b][sdx] = ((top[sdx] >> b) & 1u) ? 0xffffffffu : 0u;
    }
    *out = L.release();
    return THRML_OK;
}
void thrml_lattice_destroy(thrml_lattice* L) {
    if (!L) return;
    cudaSetDevice(L->device);
    cudaDeviceSynchronize();
    delete L;
}

int32_t thrml_lattice_set_noise(thrml_lattice* L, int32_t mapping) {
    if (!L) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    if (mapping != THRML_LATTICE_NOISE_PROGRAM && mapping != THRML_LATTICE_NOISE_PACKED && mapping != THRML_LATTICE_NOISE_PACKED_TABLE)
        return fail(THRML_ERR_INVALID_ARG, "unknown noise mapping");
    L->noise = mapping == THRML_LATTICE_NOISE_PROGRAM ? THRML_LATTICE_NOISE_PROGRAM : THRML_LATTICE_NOISE_PACKED;
    L->force_table = mapping == THRML_LATTICE_NOISE_PACKED_TABLE;
    return THRML_OK;
}
int32_t thrml_lattice_randomize(thrml_lattice* L, uint64_t key) {
    if (!L) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    CU_TRY(cudaSetDevice(L->device));
    uint64_t keys[2];
    rng_split(key, 2, keys);
    const int64_t threads = L->n_rows * L->words * (L->n_chains / 4);
    for (int c = 0; c < 2; ++c) {
        k_lattice_randomize<<<static_cast<unsigned>((threads + 127) / 128), 128, 0, L->ctx->stream>>>(L->p(c), L->W, L->row0, static_cast<int32_t>(L->n_rows), L->words,
                                                                                                    static_cast<int32_t>(L->n_chains), static_cast<uint32_t>(L->chain_offset >> 2),
                                                                                                    static_cast<uint32_t>(keys[c]), static_cast<uint32_t>(keys[c] >> 32));
        CU_TRY(cudaGetLastError());
    }
    return THRML_OK;
}

static int32_t lat_scratch(thrml_lattice* L, size_t bytes) {
    if (L->scratch.holds(bytes)) return THRML_OK;
    CU_TRY(cudaStreamSynchronize(L->ctx->stream));
    return L->scratch.alloc(bytes);
}
int32_t thrml_lattice_upload(thrml_lattice* L, const uint8_t* host) {
    if (!L || !host) return fail(THRML_ERR_INVALID_ARG, "null argument");
    CU_TRY(cudaSetDevice(L->device));
    const size_t bytes = static_cast<size_t>(L->n_chains) * L->n_rows * L->W;
    if (int32_t rc = lat_scratch(L, bytes)) return rc;
    CU_TRY(cudaMemcpyAsync(L->scratch.p, host, bytes, cudaMemcpyHostToDevice, L->ctx->stream));
    const int64_t threads = L->n_rows * L->words * L->n_chains;
    k_lattice_pack<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, L->ctx->stream>>>(static_cast<const uint8_t*>(L->scratch.p), L->p(0), L->p(1), L->W, L->row0,
                                                                                           static_cast<int32_t>(L->n_rows), L->words, static_cast<int32_t>(L->n_chains));
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaStreamSynchronize(L->ctx->stream));
    return THRML_OK;
}
int32_t thrml_lattice_download(thrml_lattice* L, uint8_t* host) {
    if (!L || !host) return fail(THRML_ERR_INVALID_ARG, "null argument");
    CU_TRY(cudaSetDevice(L->device));
    const size_t bytes = static_cast<size_t>(L->n_chains) * L->n_rows * L->W;
    if (int32_t rc = lat_scratch(L, bytes)) return rc;
    const int64_t threads = L->n_rows * L->words * L->n_chains;
    k_lattice_unpack<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, L->ctx->stream>>>(L->p(0), L->p(1), static_cast<uint8_t*>(L->scratch.p), L->W, L->row0,
                                                                                             static_cast<int32_t>(L->n_rows), L->words, static_cast<int32_t>(L->n_chains));
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaMemcpyAsync(host, L->scratch.p, bytes, cudaMemcpyDeviceToHost, L->ctx->stream));
    CU_TRY(cudaStreamSynchronize(L->ctx->stream));
    return THRML_OK;
}

// The same state as bits: host layout bits[chain][stripe row][W / 32] u32, bit k of word v = column 32 v + k (one bit per spin
// over the host link instead of one byte).
int32_t thrml_lattice_upload_bits(thrml_lattice* L, const uint32_t* host) {
    if (!L || !host) return fail(THRML_ERR_INVALID_ARG, "null argument");
    CU_TRY(cudaSetDevice(L->device));
    const size_t bytes = static_cast<size_t>(L->n_chains) * L->n_rows * (L->W / 8);
    if (int32_t rc = lat_scratch(L, bytes)) return rc;
    CU_TRY(cudaMemcpyAsync(L->scratch.p, host, bytes, cudaMemcpyHostToDevice, L->ctx->stream));
    const int64_t threads = L->n_rows * L->words * L->n_chains;
    k_lattice_pack_bits<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, L->ctx->stream>>>(static_cast<const uint32_t*>(L->scratch.p), L->p(0), L->p(1), L->row0,
                                                                                                static_cast<int32_t>(L->n_rows), L->words, static_cast<int32_t>(L->n_chains));
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaStreamSynchronize(L->ctx->stream));
    return THRML_OK;
}
int32_t thrml_lattice_download_bits(thrml_lattice* L, uint32_t* host) {
    if (!L || !host) return fail(THRML_ERR_INVALID_ARG, "null argument");
    CU_TRY(cudaSetDevice(L->device));
    const size_t bytes = static_cast<size_t>(L->n_chains) * L->n_rows * (L->W / 8);
    if (int32_t rc = lat_scratch(L, bytes)) return rc;
    const int64_t threads = L->n_rows * L->words * L->n_chains;
    k_lattice_unpack_bits<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, L->ctx->stream>>>(L->p(0), L->p(1), static_cast<uint32_t*>(L->scratch.p), L->row0,
                                                                                                  static_cast<int32_t>(L->n_rows), L->words, static_cast<int32_t>(L->n_chains));
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaMemcpyAsync(host, L->scratch.p, bytes, cudaMemcpyDeviceToHost, L->ctx->stream));
    CU_TRY(cudaStreamSynchronize(L->ctx->stream));
    return THRML_OK;
}

int32_t thrml_lattice_halo_info(thrml_lattice* L, int32_t colour, void** send_top, void** send_bottom, void** recv_top, void** recv_bottom, int64_t* row_bytes) {
    if (!L || colour < 0 || colour > 1) return fail(THRML_ERR_INVALID_ARG, "bad halo query");
    uint8_t* base = static_cast<uint8_t*>(L->plane[colour].p);
    if (send_top) *send_top = base + L->row_bytes;                       // first stripe row
    if (send_bottom) *send_bottom = base + L->row_bytes * L->n_rows;     // last stripe row
    if (recv_top) *recv_top = base;                                      // halo above the stripe
    if (recv_bottom) *recv_bottom = base + L->row_bytes * (L->n_rows + 1);
    if (row_bytes) *row_bytes = static_cast<int64_t>(L->row_bytes);
    return THRML_OK;
}
// A stripe that holds the whole lattice is its own neighbour: wrap its boundary rows into its halo rows.
int32_t thrml_lattice_wrap_halo(thrml_lattice* L, int32_t colour) {
    if (!L || colour < 0 || colour > 1) return fail(THRML_ERR_INVALID_ARG, "bad colour");
    if (L->n_rows != L->H) return fail(THRML_ERR_INVALID_ARG, "only a stripe that holds the whole lattice wraps onto itself");
    CU_TRY(cudaSetDevice(L->device));
    uint8_t* base = static_cast<uint8_t*>(L->plane[colour].p);
    CU_TRY(cudaMemcpyAsync(base, base + L->row_bytes * L->n_rows, L->row_bytes, cudaMemcpyDeviceToDevice, L->ctx->stream));
    CU_TRY(cudaMemcpyAsync(base + L->row_bytes * (L->n_rows + 1), base + L->row_bytes, L->row_bytes, cudaMemcpyDeviceToDevice, L->ctx->stream));
    return THRML_OK;
}
// Update one colour of stripe rows [row_begin, row_end) (stripe-relative).  The other colour's halo rows must hold the
// neighbouring stripes' current boundary rows.  Asynchronous on the context's stream.
int32_t thrml_lattice_update(thrml_lattice* L, int32_t colour, uint64_t block_key, int64_t row_begin, int64_t row_end) {
    if (!L || colour < 0 || colour > 1) return fail(THRML_ERR_INVALID_ARG, "bad colour");
    if (row_begin < 0 || row_end > L->n_rows || row_begin > row_end) return fail(THRML_ERR_INVALID_ARG, "row range out of the stripe");
    if (row_begin == row_end) return THRML_OK;
    CU_TRY(cudaSetDevice(L->device));
    LatArgs a{L->p(colour), L->p(1 - colour), static_cast<const uint32_t*>(L->lut.p), L->H, L->W, L->row0, static_cast<int32_t>(L->n_rows), L->words,
              static_cast<int32_t>(L->n_chains), colour, static_cast<uint32_t>(L->chain_offset >> 2), make_round_keys(block_key)};
    const int64_t threads = (row_end - row_begin) * L->words * (L->n_chains / 4);
    if (L->noise == THRML_LATTICE_NOISE_PACKED) {
        std::memcpy(a.vmask, L->vmask, sizeof(a.vmask));
        a.record = L->record_into;
        const unsigned grid = static_cast<unsigned>(std::min<int64_t>((threads + 127) / 128, static_cast<int64_t>(L->ctx->sm_count) * 12));
        const int32_t rb = static_cast<int32_t>(row_begin), re = static_cast<int32_t>(row_end);
        if (L->symmetric && !L->force_table) {
            if (a.record) k_lattice_update_sliced<true, true><<<grid, 128, 0, L->ctx->stream>>>(a, rb, re);
            else k_lattice_update_sliced<true, false><<<grid, 128, 0, L->ctx->stream>>>(a, rb, re);
        } else {
            if (a.record) k_lattice_update_sliced<false, true><<<grid, 128, 0, L->ctx->stream>>>(a, rb, re);
            else k_lattice_update_sliced<false, false><<<grid, 128, 0, L->ctx->stream>>>(a, rb, re);
        }
    } else {
        k_lattice_update<<<static_cast<unsigned>((threads + 127) / 128), 128, 0, L->ctx->stream>>>(a, static_cast<int32_t>(row_begin), static_cast<int32_t>(row_end));
    }
    CU_TRY(cudaGetLastError());
    return THRML_OK;
}
// Per chain: sum of spins and sum of bond products over this stripe (bonds counted from their colour-0 end, so stripes
// add up without double counting).  Both colours' halo rows must be current.  sums_out[2][n_chains] on the host.
int32_t thrml_lattice_observe(thrml_lattice* L, int64_t* sums_out) {
    if (!L || !sums_out) return fail(THRML_ERR_INVALID_ARG, "null argument");
    CU_TRY(cudaSetDevice(L->device));
    CU_TRY(cudaMemsetAsync(L->obs.p, 0, L->obs.bytes, L->ctx->stream));
    const int64_t cells = L->n_rows * L->words;
    const int ctas = static_cast<int>(std::min<int64_t>((cells * L->n_chains + 255) / 256, 4096));
    k_lattice_observe<<<ctas, 256, 0, L->ctx->stream>>>(L->p(0), L->p(1), L->row0, static_cast<int32_t>(L->n_rows), L->words, static_cast<int32_t>(L->n_chains),
                                                        static_cast<long long*>(L->obs.p));
    CU_TRY(cudaGetLastError());
    CU_TRY(cudaMemcpyAsync(sums_out, L->obs.p, L->obs.bytes, cudaMemcpyDeviceToHost, L->ctx->stream));
    CU_TRY(cudaStreamSynchronize(L->ctx->stream));
    return THRML_OK;
}
// Copy a boundary row of `src` (which_src: 0 = its first stripe row, 1 = its last) into a halo row of `dst` (which_dst:
// 0 = the halo above its stripe, 1 = the halo below), for one colour; device-to-device on dst's stream.  Both stripes
// must belong to lattices of the same width and chain count.  This is the halo exchange of stripes held by one process;
// stripes held by different processes exchange the same rows through the pointers of thrml_lattice_halo_info.
int32_t thrml_lattice_copy_halo(thrml_lattice* dst, int32_t which_dst, const thrml_lattice* src, int32_t which_src, int32_t colour) {
    if (!dst || !src || colour < 0 || colour > 1 || which_dst < 0 || which_dst > 1 || which_src < 0 || which_src > 1) return fail(THRML_ERR_INVALID_ARG, "bad halo copy");
    if (dst->row_bytes != src->row_bytes) return fail(THRML_ERR_INVALID_ARG, "stripes differ in width or chain count");
    CU_TRY(cudaSetDevice(dst->device));
    uint8_t* d = static_cast<uint8_t*>(dst->plane[colour].p) + (which_dst ? dst->row_bytes * (dst->n_rows + 1) : 0);
    const uint8_t* s_ = static_cast<const uint8_t*>(src->plane[colour].p) + (which_src ? src->row_bytes * src->n_rows : src->row_bytes);
    CU_TRY(cudaMemcpyAsync(d, s_, dst->row_bytes, cudaMemcpyDeviceToDevice, dst->ctx->stream));
    return THRML_OK;
}
// ---------------------------------------------------------------------------------------------------------
// Sweep driver inside the library (run_blocks, sampling.rs:81-106, over sample_blocks, sampling.rs:28-63).
// ---------------------------------------------------------------------------------------------------------
static int32_t lat_update_rows(thrml_lattice* L, int32_t colour, uint64_t block_key, int64_t r0, int64_t r1) { return thrml_lattice_update(L, colour, block_key, r0, r1); }

// This stripe's first row of `colour` goes to the stripe above (into its lower halo), its last row to the stripe below
// (into its upper halo); the matching rows arrive from both.  One NCCL group on `st`.  With two stripes both neighbours
// are the same rank and messages between one pair match in issue order, so the receives are posted in the order the
// peer sends: its first row (this stripe's lower halo), then its last row (this stripe's upper halo).
static int32_t lat_exchange(thrml_lattice* L, int32_t colour, thrml_comm* comm, cudaStream_t st) {
    const NcclApi* api = nccl_api();
    if (!api) return THRML_ERR_NCCL;
    uint8_t* base = static_cast<uint8_t*>(L->plane[colour].p);
    const int up = (comm->rank + comm->world - 1) % comm->world, down = (comm->rank + 1) % comm->world;
    NCCL_TRY(api, GroupStart());
    NCCL_TRY(api, Send(base + L->row_bytes, L->row_bytes, ncclUint8, up, comm->nccl, st));
    NCCL_TRY(api, Send(base + L->row_bytes * L->n_rows, L->row_bytes, ncclUint8, down, comm->nccl, st));
    NCCL_TRY(api, Recv(base + L->row_bytes * (L->n_rows + 1), L->row_bytes, ncclUint8, down, comm->nccl, st));
    NCCL_TRY(api, Recv(base, L->row_bytes, ncclUint8, up, comm->nccl, st));
    NCCL_TRY(api, GroupEnd());
    return THRML_OK;
}
static int32_t lat_check_comm(const thrml_lattice* L, const thrml_comm* comm) {
    const bool whole = L->n_rows == L->H;
    if (!comm || comm->world == 1) {
        if (!whole) return fail(THRML_ERR_INVALID_ARG, "a stripe that holds part of the lattice needs a communicator for its halo rows");
        return THRML_OK;
    }
    if (comm->ctx != L->ctx) return fail(THRML_ERR_INVALID_ARG, "communicator and lattice belong to different contexts");
    if (whole || L->H % comm->world || L->n_rows != L->H / comm->world || L->row0 != comm->rank * L->n_rows)
        return fail(THRML_ERR_INVALID_ARG, "with a communicator, rank r must hold rows [r * H / world, (r + 1) * H / world)");
    return THRML_OK;
}
static int32_t lat_refresh_halos(thrml_lattice* L, int32_t colour, thrml_comm* comm) {
    if (!comm || comm->world == 1) return thrml_lattice_wrap_halo(L, colour);
    return lat_exchange(L, colour, comm, L->ctx->stream);
}
// Next free record of the observable series (zeroed), growing the buffer when it is full.
static int32_t lat_next_record(thrml_lattice* L, long long** slot) {
    const size_t rec = static_cast<size_t>(2 * L->n_chains) * 8;
    if (L->series_len == L->series_cap) {  // grow, keeping the records
        const int64_t cap = std::max<int64_t>(1024, 2 * L->series_cap);
        DevBuf bigger;
        if (int32_t rc = bigger.alloc(static_cast<size_t>(cap) * rec)) return rc;
        CU_TRY(cudaMemsetAsync(bigger.p, 0, bigger.bytes, L->ctx->stream));
        if (L->series_len > 0) CU_TRY(cudaMemcpyAsync(bigger.p, L->series.p, static_cast<size_t>(L->series_len) * rec, cudaMemcpyDeviceToDevice, L->ctx->stream));
        CU_TRY(cudaStreamSynchronize(L->ctx->stream));
        std::swap(L->series.p, bigger.p);
        std::swap(L->series.bytes, bigger.bytes);
        L->series_cap = cap;
    }
    *slot = static_cast<long long*>(L->series.p) + L->series_len * 2 * L->n_chains;
    ++L->series_len;
    return THRML_OK;
}
// The observable kernel on its own (noise mapping 0, whose update kernel does not record).
static int32_t lat_observe_into(thrml_lattice* L, long long* slot) {
    const int64_t cells = L->n_rows * L->words;
    const int ctas = static_cast<int>(std::min<int64_t>((cells * L->n_chains + 255) / 256, 4096));
    k_lattice_observe<<<ctas, 256, 0, L->ctx->stream>>>(L->p(0), L->p(1), L->row0, static_cast<int32_t>(L->n_rows), L->words, static_cast<int32_t>(L->n_chains), slot);
    CU_TRY(cudaGetLastError());
    return THRML_OK;
}

int32_t thrml_lattice_refresh_halos(thrml_lattice* L, thrml_comm* comm) {
    if (!L) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    if (int32_t rc = lat_check_comm(L, comm)) return rc;
    CU_TRY(cudaSetDevice(L->device));
    for (int colour = 0; colour < 2; ++colour)
        if (int32_t rc = lat_refresh_halos(L, colour, comm)) return rc;
    return THRML_OK;
}

int32_t thrml_lattice_run_blocks(thrml_lattice* L, uint64_t key, int64_t n_iters, thrml_comm* comm, int32_t record) {
    if (!L) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    if (n_iters < 0) return fail(THRML_ERR_INVALID_ARG, "n_iters must be non-negative");
    if (int32_t rc = lat_check_comm(L, comm)) return rc;
    CU_TRY(cudaSetDevice(L->device));
    const bool dist = comm && comm->world > 1;
    const bool overlap = dist && L->n_rows >= 4;
    if (overlap && !L->side) {
        CU_TRY(cudaStreamCreateWithFlags(&L->side, cudaStreamNonBlocking));
        CU_TRY(cudaEventCreateWithFlags(&L->ev_edge, cudaEventDisableTiming));
        CU_TRY(cudaEventCreateWithFlags(&L->ev_halo, cudaEventDisableTiming));
    }
    cudaStream_t st = L->ctx->stream;
    std::vector<uint64_t> keys(static_cast<size_t>(n_iters));
    rng_split(key, n_iters, keys.data());  // run_blocks: key.split(n_iters)
    struct ClearRecord {  // no later per-colour call may inherit the record pointer, whichever way this function returns
        thrml_lattice* lat;
        ~ClearRecord() { lat->record_into = nullptr; }
    } clear_record{L};
    const bool fused_record = record && L->noise == THRML_LATTICE_NOISE_PACKED;  // that mapping's update kernel records while it updates
    for (int64_t it = 0; it < n_iters; ++it) {
        uint64_t k2[2];
        rng_split(keys[it], 2, k2);  // sample_blocks: one key per free block
        long long* slot = nullptr;
        if (record)
            if (int32_t rc = lat_next_record(L, &slot)) return rc;
        for (int colour = 0; colour < 2; ++colour) {
            // the second colour's pass sees every bond and every word of the first colour exactly once
            L->record_into = fused_record && colour == 1 ? slot : nullptr;
            if (!overlap) {
                if (int32_t rc = lat_update_rows(L, colour, k2[colour], 0, L->n_rows)) return rc;
                if (int32_t rc = lat_refresh_halos(L, colour, comm)) return rc;
                continue;
            }
            // boundary rows first; they travel on the side stream while the interior rows are updated
            if (int32_t rc = lat_update_rows(L, colour, k2[colour], 0, 1)) return rc;
            if (int32_t rc = lat_update_rows(L, colour, k2[colour], L->n_rows - 1, L->n_rows)) return rc;
            CU_TRY(cudaEventRecord(L->ev_edge, st));
            CU_TRY(cudaStreamWaitEvent(L->side, L->ev_edge, 0));
            if (int32_t rc = lat_exchange(L, colour, comm, L->side)) return rc;
            CU_TRY(cudaEventRecord(L->ev_halo, L->side));
            if (int32_t rc = lat_update_rows(L, colour, k2[colour], 1, L->n_rows - 1)) return rc;
            CU_TRY(cudaStreamWaitEvent(st, L->ev_halo, 0));  // the other colour reads these halo rows next
        }
        L->record_into = nullptr;
        if (record && !fused_record)
            if (int32_t rc = lat_observe_into(L, slot)) return rc;
    }
    return THRML_OK;
}

int32_t thrml_lattice_series_reset(thrml_lattice* L) {
    if (!L) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    CU_TRY(cudaSetDevice(L->device));
    if (L->series.p) CU_TRY(cudaMemsetAsync(L->series.p, 0, L->series.bytes, L->ctx->stream));
    L->series_len = 0;
    return THRML_OK;
}

// The recorded series summed over the stripes of `comm` (one allreduce of the whole series), on the host:
// series_out[record][2][chain] int64 = (sum of spins, sum of bond products) of the whole lattice after each recorded sweep.
int32_t thrml_lattice_read_series(thrml_lattice* L, thrml_comm* comm, int64_t* series_out, int64_t capacity_records, int64_t* n_records_out) {
    if (!L) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    if (int32_t rc = lat_check_comm(L, comm)) return rc;
    if (n_records_out) *n_records_out = L->series_len;
    if (!series_out || L->series_len == 0) return THRML_OK;
    if (capacity_records < L->series_len) return fail(THRML_ERR_INVALID_ARG, "series buffer holds fewer records than were recorded");
    CU_TRY(cudaSetDevice(L->device));
    const size_t count = static_cast<size_t>(L->series_len) * 2 * L->n_chains;
    const void* src = L->series.p;
    if (comm && comm->world > 1) {
        const NcclApi* api = nccl_api();
        if (!api) return THRML_ERR_NCCL;
        if (int32_t rc = lat_scratch(L, count * 8)) return rc;
        NCCL_TRY(api, AllReduce(L->series.p, L->scratch.p, count, ncclInt64, ncclSum, comm->nccl, L->ctx->stream));
        src = L->scratch.p;
    }
    CU_TRY(cudaMemcpyAsync(series_out, src, count * 8, cudaMemcpyDeviceToHost, L->ctx->stream));
    CU_TRY(cudaStreamSynchronize(L->ctx->stream));
    return THRML_OK;
}

// First and second moments over the recorded sweeps of the magnetisation per spin m = sum s / N and the energy per spin
// e = -(J sum_bonds s_i s_j + b sum s) / N (J, b without beta): moments_out[4][chain] = <m>, <m^2>, <e>, <e^2>.
int32_t thrml_lattice_moments(thrml_lattice* L, thrml_comm* comm, double* moments_out, int64_t* n_records_out) {
    if (!L || !moments_out) return fail(THRML_ERR_INVALID_ARG, "null argument");
    std::vector<int64_t> series(static_cast<size_t>(std::max<int64_t>(L->series_len, 1)) * 2 * L->n_chains);
    int64_t n = 0;
    if (int32_t rc = thrml_lattice_read_series(L, comm, series.data(), L->series_len, &n)) return rc;
    if (n_records_out) *n_records_out = n;
    const double N = static_cast<double>(L->H) * static_cast<double>(L->W);
    for (int64_t c = 0; c < L->n_chains; ++c) {
        double m1 = 0, m2 = 0, e1 = 0, e2 = 0;
        for (int64_t t = 0; t < n; ++t) {
            const double S = static_cast<double>(series[(t * 2 + 0) * L->n_chains + c]), B = static_cast<double>(series[(t * 2 + 1) * L->n_chains + c]);
            const double m = S / N, e = -(static_cast<double>(L->coupling) * B + static_cast<double>(L->bias) * S) / N;
            m1 += m; m2 += m * m; e1 += e; e2 += e * e;
        }
        const double inv = n > 0 ? 1.0 / static_cast<double>(n) : 0.0;
        moments_out[0 * L->n_chains + c] = m1 * inv;
        moments_out[1 * L->n_chains + c] = m2 * inv;
        moments_out[2 * L->n_chains + c] = e1 * inv;
        moments_out[3 * L->n_chains + c] = e2 * inv;
    }
    return THRML_OK;
}

int32_t thrml_lattice_synchronize(thrml_lattice* L) {
    if (!L) return fail(THRML_ERR_INVALID_ARG, "null lattice");
    CU_TRY(cudaSetDevice(L->device));
    CU_TRY(cudaStreamSynchronize(L->ctx->stream));
    return THRML_OK;
}

}  // extern "C"
