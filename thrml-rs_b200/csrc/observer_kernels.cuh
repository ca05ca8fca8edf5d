// Initialisation, layout conversion, observers (moments, marginals, bit-packed rows) and per-chain energies.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "device_math.cuh"

using namespace thrml;

// hinton_init (ising.rs:602-673) and uniform start.  One thread = one node x four chains.
__global__ void __launch_bounds__(256) k_hinton(uint8_t* dst, int64_t ld, int64_t n_chains, int32_t n, const float* bias, float beta,
                                                uint32_t chain_word0, uint32_t k0, uint32_t k1, const float* inj) {
    const int quad = blockIdx.y * blockDim.x + threadIdx.x;
    const int node = blockIdx.x * blockDim.y + threadIdx.y;
    if (node >= n || 4 * static_cast<int64_t>(quad) >= ld) return;
    const float p = det_sigmoid(__fmul_rn(bias[node], beta));  // ising.rs:650
    const U4 r = philox4x32_10(static_cast<uint32_t>(node), chain_word0 + static_cast<uint32_t>(quad), 0u, TAG_HINT, k0, k1);
    uint32_t out = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int64_t chain = 4 * static_cast<int64_t>(quad) + c;
        if (chain >= n_chains) continue;
        const float u = inj ? inj[chain * n + node] : u24(pick(r, c));
        if (u <= p) out |= 1u << (8 * c);  // ising.rs:667
    }
    *reinterpret_cast<uint32_t*>(dst + static_cast<int64_t>(node) * ld + 4 * static_cast<int64_t>(quad)) = out;
}
__global__ void __launch_bounds__(256) k_randomize(uint8_t* dst, int64_t ld, int64_t n_chains, int32_t n, int32_t kind, uint32_t chain_word0,
                                                   uint32_t k0, uint32_t k1) {
    const int quad = blockIdx.y * blockDim.x + threadIdx.x;
    const int node = blockIdx.x * blockDim.y + threadIdx.y;
    if (node >= n || 4 * static_cast<int64_t>(quad) >= ld) return;
    const U4 r = philox4x32_10(static_cast<uint32_t>(node), chain_word0 + static_cast<uint32_t>(quad), 0u, TAG_RAND, k0, k1);
    uint32_t out = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        if (4 * static_cast<int64_t>(quad) + c >= n_chains) continue;
        const uint32_t x = pick(r, c);
        const uint32_t v = kind == 0 ? (x >> 31) : static_cast<uint32_t>((static_cast<uint64_t>(x >> 8) * static_cast<uint64_t>(kind)) >> 24);
        out |= v << (8 * c);
    }
    *reinterpret_cast<uint32_t*>(dst + static_cast<int64_t>(node) * ld + 4 * static_cast<int64_t>(quad)) = out;
}

// [chain][node] (host order) <-> [node][chain] (device order), through a 32x32 shared-memory tile.
__global__ void k_transpose_in(const uint8_t* src, uint8_t* dst, int64_t n, int64_t n_chains, int64_t ld) {
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
__global__ void k_transpose_out(const uint8_t* src, uint8_t* dst, int64_t n, int64_t n_chains, int64_t ld) {
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

// Moment observer (moment.rs:205-233): per row the product of f(x) over its members, summed over chains.
// One warp-row = one moment row; lanes stride over chain words; exact int64 accumulation.
__global__ void __launch_bounds__(256) k_moments(const int64_t* row_ptr, const int32_t* mem_sd, const int32_t* mem_pos, int64_t n_rows,
                                                 const uint8_t* cls0, const uint8_t* cls1, int64_t ld, int64_t n_chains, int32_t spin_transform,
                                                 unsigned long long* sums, const int64_t* row_ids) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + threadIdx.y;
    if (row >= n_rows) return;
    const int64_t b = row_ptr[row], e = row_ptr[row + 1];
    long long acc = 0;
    for (int64_t quad = threadIdx.x; 4 * quad < n_chains; quad += 32) {
        long long prod[4] = {1, 1, 1, 1};
        for (int64_t q = b; q < e; ++q) {
            const uint8_t* base = mem_sd[q] == 0 ? cls0 : cls1;
            const uint32_t wd = *reinterpret_cast<const uint32_t*>(base + static_cast<int64_t>(mem_pos[q]) * ld + 4 * quad);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const long long x = (wd >> (8 * c)) & 0xffu;
                prod[c] *= spin_transform ? 2 * x - 1 : x;
            }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
            if (4 * quad + c < n_chains) acc += prod[c];
    }
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, off);
    if (threadIdx.x == 0) atomicAdd(sums + (row_ids ? row_ids[row] : row), static_cast<unsigned long long>(acc));
}
// The same observer for rows whose members are all spins read as +-1 (the Ising moment spec, moment.rs:125-148): the
// product of (2x - 1) over a row is -1 exactly when an odd number of members is 0, so one XOR per member and one
// population count per word replace the per-chain products.  One warp per row, 16 chains per lane per pass.
__global__ void __launch_bounds__(256) k_moments_spin(const int64_t* row_ptr, const int32_t* mem_pos, int64_t n_rows, const uint8_t* spin, int64_t ld, int64_t n_chains,
                                                      unsigned long long* sums, const int64_t* row_ids) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + threadIdx.y;
    if (row >= n_rows) return;
    const int64_t b = row_ptr[row], e = row_ptr[row + 1];
    const int64_t n_chunks = (n_chains + 15) / 16;
    int odd = 0;  // chains whose row has an odd number of zeros
    for (int64_t ch = threadIdx.x; ch < n_chunks; ch += 32) {
        uint4 z = make_uint4(0, 0, 0, 0);
        for (int64_t q = b; q < e; ++q) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(spin + static_cast<int64_t>(mem_pos[q]) * ld) + ch);
            z.x ^= ~v.x; z.y ^= ~v.y; z.z ^= ~v.z; z.w ^= ~v.w;
        }
        const uint32_t wd[4] = {z.x, z.y, z.z, z.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t left = n_chains - (16 * ch + 4 * k);  // chains beyond the last one do not count
            const uint32_t vm = left >= 4 ? 0x01010101u : (left <= 0 ? 0u : (0x01010101u >> (8 * (4 - static_cast<int>(left)))));
            odd += __popc(wd[k] & vm);
        }
    }
    odd = __reduce_add_sync(0xffffffffu, odd);
    if (threadIdx.x == 0) atomicAdd(sums + (row_ids ? row_ids[row] : row), static_cast<unsigned long long>(static_cast<long long>(n_chains) - 2ll * odd));
}
// Category counts per observed node.
__global__ void __launch_bounds__(256) k_marginals(const int32_t* node_sd, const int32_t* node_pos, int64_t n_nodes, int32_t K, const uint8_t* cls0,
                                                   const uint8_t* cls1, int64_t ld, int64_t n_chains, unsigned long long* counts) {
    const int64_t node = static_cast<int64_t>(blockIdx.x) * 8 + threadIdx.y;
    if (node >= n_nodes) return;
    const uint8_t* row = (node_sd[node] == 0 ? cls0 : cls1) + static_cast<int64_t>(node_pos[node]) * ld;
    for (int cat = 0; cat < K; ++cat) {
        int cnt = 0;
        for (int64_t chain = threadIdx.x; chain < n_chains; chain += 32) cnt += row[chain] == cat;
        for (int off = 16; off > 0; off >>= 1) cnt += __shfl_down_sync(0xffffffffu, cnt, off);
        if (threadIdx.x == 0 && cnt) atomicAdd(counts + node * K + cat, static_cast<unsigned long long>(cnt));
    }
}

// Ising energy per chain, E = -beta (sum b_i s_i + sum J_ij s_i s_j) (ising.rs:227-321), in f64.  Terms are cut into
// chunks; each CTA sums one chunk for 128 chains (8 term lanes x 32 chain quads, combined in a fixed order), a second
// pass adds the chunks in order, so the result does not depend on scheduling.
constexpr int ENERGY_CHUNK = 2048;
__global__ void __launch_bounds__(256) k_energy_partial(const int32_t* pos_a, const int32_t* pos_b, const float* w, int64_t n_terms, const uint8_t* spin, int64_t ld,
                                                        int64_t n_chains, double* partial /*[chunks][ld]*/) {
    __shared__ double red[8][32][4];
    const int64_t quad = static_cast<int64_t>(blockIdx.y) * 32 + threadIdx.x;
    const int64_t t0 = static_cast<int64_t>(blockIdx.x) * ENERGY_CHUNK, t1 = min(n_terms, t0 + ENERGY_CHUNK);
    double acc[4] = {0.0, 0.0, 0.0, 0.0};
    if (4 * quad < ld) {
        for (int64_t t = t0 + threadIdx.y; t < t1; t += 8) {
            const uint32_t a = *reinterpret_cast<const uint32_t*>(spin + static_cast<int64_t>(pos_a[t]) * ld + 4 * quad);
            const int32_t pb = pos_b[t];
            const uint32_t b = pb >= 0 ? *reinterpret_cast<const uint32_t*>(spin + static_cast<int64_t>(pb) * ld + 4 * quad) : 0x01010101u;
            const double wt = static_cast<double>(w[t]);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t agree = ~(a ^ b) >> (8 * c) & 1u;  // s_a s_b = +1 when the bits agree
                acc[c] += agree ? wt : -wt;
            }
        }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) red[threadIdx.y][threadIdx.x][c] = acc[c];
    __syncthreads();
    if (threadIdx.y == 0 && 4 * quad < ld) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            double sum = 0.0;
            for (int y = 0; y < 8; ++y) sum += red[y][threadIdx.x][c];
            partial[static_cast<int64_t>(blockIdx.x) * ld + 4 * quad + c] = sum;
        }
    }
}
// DiscreteEBMFactor::factor_energy (discrete_ebm.rs:552-592) for every chain: sum over rows of
// W[row][c1][c2] * prod over spin groups of (2x - 1), in f64, with the chunking of k_energy_partial.
// pos: [n_spin + n_cat][n_terms] positions in the spin / categorical class arrays.
__global__ void __launch_bounds__(256) k_factor_energy_partial(const int32_t* pos, int32_t n_spin, int32_t n_cat, const float* w, int32_t d1, int32_t d2, int64_t n_terms,
                                                               const uint8_t* spin, const uint8_t* cat, int64_t ld, double* partial /*[chunks][ld]*/) {
    __shared__ double red[8][32][4];
    const int64_t quad = static_cast<int64_t>(blockIdx.y) * 32 + threadIdx.x;
    const int64_t t0 = static_cast<int64_t>(blockIdx.x) * ENERGY_CHUNK, t1 = min(n_terms, t0 + ENERGY_CHUNK);
    double acc[4] = {0.0, 0.0, 0.0, 0.0};
    if (4 * quad < ld) {
        for (int64_t t = t0 + threadIdx.y; t < t1; t += 8) {
            uint32_t zeros = 0;  // per chain byte: parity of the number of spin tails that are 0 (each contributes a factor -1)
            for (int32_t g = 0; g < n_spin; ++g)
                zeros ^= ~*reinterpret_cast<const uint32_t*>(spin + static_cast<int64_t>(pos[g * n_terms + t]) * ld + 4 * quad);
            uint32_t c1 = 0, c2 = 0;
            if (n_cat > 0) c1 = *reinterpret_cast<const uint32_t*>(cat + static_cast<int64_t>(pos[n_spin * n_terms + t]) * ld + 4 * quad);
            if (n_cat > 1) c2 = *reinterpret_cast<const uint32_t*>(cat + static_cast<int64_t>(pos[(n_spin + 1) * n_terms + t]) * ld + 4 * quad);
            const float* wt = w + t * d1 * d2;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int32_t i1 = min(static_cast<int32_t>((c1 >> (8 * c)) & 0xffu), d1 - 1), i2 = min(static_cast<int32_t>((c2 >> (8 * c)) & 0xffu), d2 - 1);
                const double v = static_cast<double>(wt[i1 * d2 + i2]);
                acc[c] += ((zeros >> (8 * c)) & 1u) ? -v : v;
            }
        }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) red[threadIdx.y][threadIdx.x][c] = acc[c];
    __syncthreads();
    if (threadIdx.y == 0 && 4 * quad < ld) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            double sum = 0.0;
            for (int y = 0; y < 8; ++y) sum += red[y][threadIdx.x][c];
            partial[static_cast<int64_t>(blockIdx.x) * ld + 4 * quad + c] = sum;
        }
    }
}
__global__ void k_energy_final(const double* partial, int64_t n_chunks, int64_t ld, int64_t n_chains, double neg_beta, double* out) {
    const int64_t chain = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (chain >= n_chains) return;
    double sum = 0.0;
    for (int64_t k = 0; k < n_chunks; ++k) sum += partial[k * ld + chain];
    out[chain] = neg_beta * sum;
}

// Bit-packs spin rows for streaming to the host: out[row][word] bit (c & 31) = state of chain 32*word + c.
// One warp per (row, group of 32 words); a ballot turns 32 chains into one word.
__global__ void __launch_bounds__(256) k_pack_rows(const uint8_t* rows, int64_t ld, int64_t n_chains, int64_t n_rows, int64_t words, uint32_t* out) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + threadIdx.y;
    if (row >= n_rows) return;
    for (int64_t wd = 0; wd < words; ++wd) {
        const int64_t chain = 32 * wd + threadIdx.x;
        const uint32_t bit = chain < n_chains ? (rows[row * ld + chain] & 1u) : 0u;
        const uint32_t word = __ballot_sync(0xffffffffu, bit);
        if (threadIdx.x == 0) out[row * words + wd] = word;
    }
}

// The inverse of k_pack_rows, for uploads: in[row][word] bit (c & 31) -> one byte per chain.  One thread expands 16
// chains (one 16-byte store); chains beyond n_chains are written as zero.
__global__ void __launch_bounds__(256) k_unpack_rows(const uint32_t* in, int64_t words, int64_t n_rows, int64_t ld, int64_t n_chains, uint8_t* rows) {
    const int64_t chunks = ld >> 4;
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= n_rows * chunks) return;
    const int64_t row = gid / chunks, chunk = gid % chunks;
    uint32_t bits = (__ldg(in + row * words + (chunk >> 1)) >> (16 * static_cast<int>(chunk & 1))) & 0xffffu;
    const int64_t left = n_chains - 16 * chunk;
    if (left < 16) bits &= left > 0 ? ((1u << static_cast<int>(left)) - 1u) : 0u;
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint32_t nib = (bits >> (4 * q)) & 15u;
        w[q] = (nib & 1u) | ((nib & 2u) << 7) | ((nib & 4u) << 14) | ((nib & 8u) << 21);
    }
    *reinterpret_cast<uint4*>(rows + row * ld + 16 * chunk) = make_uint4(w[0], w[1], w[2], w[3]);
}

// int64 <-> int32 views of the moment sums for the allreduce (used only when every total provably fits 32 bits).
__global__ void k_narrow_i64(const long long* src, int32_t* dst, int64_t n) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = static_cast<int32_t>(src[i]);
}
__global__ void k_widen_i32(const int32_t* src, long long* dst, int64_t n) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = static_cast<long long>(src[i]);
}
