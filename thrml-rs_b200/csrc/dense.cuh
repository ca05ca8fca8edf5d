// Dense bipartite path: tcgen05 tensor-core GEMMs with TMEM accumulators, operands staged by TMA.
//
// A spin block whose every neighbour lies in one other block (an RBM layer) has the local field
//     gamma[chain][i] = bias[i] + sum_j W[i][j] * (2 s[chain][j] - 1)            (spin_gibbs.rs:512-611 for a complete bipartite table)
// which is the GEMM  D[chains x n_out] = S[chains x n_in] * W^T  with S = +-1 in bf16 and W in bf16, f32 accumulation.
// k_dense_gemm<EPI_SAMPLE> runs that GEMM and finishes each output tile in registers: bias, sigmoid, counter-based noise
// under this path's own key -> noise mapping (one generator call gives a lane the top halves of eight draws of its chain),
// Bernoulli draw, and stores of the new state (bytes, engine layout) and of its +-1 bf16 image (the next layer's S operand).
// k_dense_gemm<EPI_CORR> computes pair correlations <s_a s_b> over chains straight from the engine's byte state
// (0/1 bytes, chains contiguous = K-major) with the 8-bit integer MMA: N11 = sum_c x_a x_b, then
// sum_c s_a s_b = 4 N11 - 2 N1a - 2 N1b + C exactly.
//
// One CTA per SM, persistent over output tiles.  Warp 0: TMA producer.  Warp 1: MMA issuer and TMEM owner.
// Warps 2-17: epilogue; a warp reads the 32 TMEM lanes its warp index modulo 4 selects, and the four warps that share a
// lane quarter split the tile's columns.  Sixteen epilogue warps keep four warps on every scheduler: with fewer the
// per-element math (noise, sigmoid, compare) runs at dependent-issue latency and hides the tensor pipe behind it.
// Shared-memory stages and the two TMEM accumulators are handed over through mbarriers; every wait is bounded and
// reports through an error flag.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "device_math.cuh"

namespace thrml {
namespace dense {

constexpr int BM = 128;          // tile rows (TMEM lanes)
constexpr int BK_BYTES = 128;    // one 128-byte swizzle atom along K per stage
constexpr int STAGE_BUDGET = 192 * 1024;  // shared memory spent on operand stages
constexpr int ACC_BUFS = 2;
constexpr int EPI_WARPS = 16;
constexpr int THREADS = 64 + 32 * EPI_WARPS;
constexpr uint32_t SPIN_LIMIT = 1u << 24;  // hard cap on the number of parked waits of one mbar_wait (the time bound normally ends it first)

enum Epilogue { EPI_SAMPLE = 0, EPI_CORR = 1, EPI_FIELDS = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait on a phase parity.  Returns false (and raises *err) when the limit runs out.
// try_wait parks the thread in hardware for up to the hinted time instead of spinning: a polling loop in the producer
// or MMA warp would take issue slots from the epilogue warps that share its scheduler.  The bound is wall time
// (about two seconds on the global nanosecond timer), checked between the parked waits.
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err, int code) {
    const uint32_t addr = smem_u32(bar);
    uint64_t t0 = 0;
    for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity), "r"(20000u)
            : "memory");
        if (ok) return true;
        if ((spin & 15u) == 15u) {
            if (*reinterpret_cast<volatile int*>(err) != 0) return false;  // another role gave up
            const uint64_t now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_LIMIT_NS) break;
        }
    }
    atomicCAS(err, 0, code);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, uint64_t* bar, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes, 128-byte swizzled, groups of 8 rows
// 1024 bytes apart: start address, leading offset 16 B (unused for this layout), stride offset 1024 B, descriptor
// version 1, layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}
// Instruction descriptor: accumulator format (1 f32, 2 s32), A/B formats, both K-major, N/8 at bit 17, M/16 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t c_fmt, uint32_t ab_fmt, uint32_t m, uint32_t n) {
    return (c_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

template <int KIND_I8>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if (KIND_I8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Asynchronous TMEM load of 16 columns of this thread's lane; the registers are valid after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct GemmArgs {
    int32_t m_total, n_total, k_bytes;  // problem size; k in bytes along the contiguous dimension
    int32_t tiles_m, tiles_n;
    int* err;
    // EPI_SAMPLE
    const float* bias;        // [n_total]
    uint8_t* state_out;       // first state row of the updated block, [n_total][ld]
    int64_t ld;
    __nv_bfloat16* image_out; // +-1 bf16 image [m_total rows = chains][image_pitch], or null
    int64_t image_pitch;      // elements
    uint32_t chain_word0;
    PhiloxRoundKeys rk;       // round keys of the block key
    int32_t* ones_out;        // [n_total] number of ones per updated node, accumulated with atomics (zeroed by the caller), or null
    // EPI_CORR
    const int32_t* ones_a;    // [m_total] number of ones per row of A
    const int32_t* ones_b;    // [n_total]
    float* corr_out;          // [m_total][n_total], or [n_total][m_total] when corr_transposed
    int32_t n_chains;
    int32_t corr_transposed;
    uint32_t* debug;          // nullable: the pair kernel records each CTA's TMEM base address here
    // EPI_FIELDS
    float* fields_out;        // [m_total = chains][n_total]: bias + accumulator, the local field the sampling epilogue would draw from
};

// Finishes 16 accumulator columns of one warp's 32 rows: `acc` holds this lane's row (row_base + lane), columns
// col0..col0+15 of the whole problem.
template <int EPI>
__device__ __forceinline__ void finish_chunk(const GemmArgs& g, uint32_t (&acc)[16], int row_base, int col0, int lane) {
    const int row = row_base + lane;
    if (EPI == EPI_SAMPLE) {
        // row = chain, columns = nodes of the updated block
        float bias[16];
        if (col0 + 16 <= g.n_total) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 b4 = __ldg(reinterpret_cast<const float4*>(g.bias + col0) + q);
                bias[4 * q] = b4.x; bias[4 * q + 1] = b4.y; bias[4 * q + 2] = b4.z; bias[4 * q + 3] = b4.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) bias[j] = col0 + j < g.n_total ? __ldg(g.bias + col0 + j) : 0.0f;
        }
        // Noise of the dense path (its own key -> noise mapping; the reference never consumes its keys).  The 32-bit draw of
        // node n and global chain c is
        //     top 16 bits = half (n & 1) of word ((n >> 1) & 3) of Philox(n >> 3, c, 1, TAG_SPIN)   -- one call: 8 nodes of one chain
        //     low 16 bits = low half of word (c & 3) of Philox(n, c >> 2, 2, TAG_SPIN)
        // and the spin is 1 iff the draw's top 24 bits, as a uniform, are <= sigmoid(2 gamma).  A lane owns one chain and 16
        // consecutive nodes here, so two calls give it every top half it needs and nothing crosses lanes; the low half is
        // fetched only for a draw whose top half cannot decide.
        const uint32_t chain = 4u * g.chain_word0 + static_cast<uint32_t>(row);
        uint32_t top[16];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const U4 r = philox4x32_10_rk(static_cast<uint32_t>(col0 >> 3) + t, chain, 1u, TAG_SPIN, g.rk);
            const uint32_t wds[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                top[8 * t + 2 * i] = wds[i] & 0xffffu;
                top[8 * t + 2 * i + 1] = wds[i] >> 16;
            }
        }
        // d = 2^16 (u_top - p) with the approximate sigmoid p = 1 / (1 + 2^(-2 log2(e) gamma)), as top - 1 / (2^-16 (1 + e))
        // (a huge exponential gives p = 0, a vanishing one p = 1).  The full uniform lies in [top, top + 1) 2^-16, so the spin is
        // 1 for d <= -1 and 0 for d >= 0 once the approximation's error (below 0.3 of these units: four times its worst 1e-6)
        // is allowed for; inside (-1.3, 0.3) the low half is drawn and the exact sigmoid decides.  The decisions stay in the
        // sign bits of d: no per-element bit masks are built.
        constexpr float ZONE_MID = 0.5f, ZONE_HALF = 0.8f;
        float d[16];
        float nearest = 65536.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float gamma = __fadd_rn(bias[j], __uint_as_float(acc[j]));
            float e, p16;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(gamma * -2.885390081777927f));
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(p16) : "f"(fmaf(e, 1.52587890625e-5f, 1.52587890625e-5f)));
            d[j] = __uint2float_rn(top[j]) - p16;
            nearest = fminf(nearest, fabsf(d[j] + ZONE_MID));
        }
        if (__any_sync(0xffffffffu, nearest <= ZONE_HALF)) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (fabsf(d[j] + ZONE_MID) <= ZONE_HALF) {
                    const U4 rr = philox4x32_10_rk(static_cast<uint32_t>(col0 + j), chain >> 2, 2u, TAG_SPIN, g.rk);
                    const uint32_t draw = (top[j] << 16) | (pick(rr, chain & 3u) & 0xffffu);
                    const float xx = __fmul_rn(__fadd_rn(bias[j], __uint_as_float(acc[j])), 2.0f);
                    d[j] = u24(draw) <= det_sigmoid(xx) ? -1.0f : 1.0f;
                }
        }
        // state bytes: lane L takes column L&15 and the 16 chains of half L>>4 of this warp's 32 rows
        const uint32_t live = row_base + 32 <= g.m_total ? 0xffffffffu : (row_base < g.m_total ? 0xffffffffu >> (32 - (g.m_total - row_base)) : 0u);
        uint32_t mine = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t m = __ballot_sync(0xffffffffu, d[j] < 0.0f);
            if ((lane & 15) == j) mine = m;
        }
        mine &= live;  // rows beyond the last chain hold no state
        {
            const int col = col0 + (lane & 15);
            const uint32_t half = (mine >> (16 * (lane >> 4))) & 0xffffu;
            if (col < g.n_total && row_base < g.m_total) {
                uint4 v;
                v.x = ((half & 0xfu) * 0x00204081u) & 0x01010101u;
                v.y = (((half >> 4) & 0xfu) * 0x00204081u) & 0x01010101u;
                v.z = (((half >> 8) & 0xfu) * 0x00204081u) & 0x01010101u;
                v.w = (((half >> 12) & 0xfu) * 0x00204081u) & 0x01010101u;
                uint8_t* dst = g.state_out + static_cast<int64_t>(col) * g.ld + row_base + 16 * (lane >> 4);
                if (row_base + 16 * (lane >> 4) < g.ld) *reinterpret_cast<uint4*>(dst) = v;  // ld is a multiple of 16
                if (g.ones_out && (lane >> 4) == 0) atomicAdd(g.ones_out + col, __popc(mine));
            }
        }
        if (row < g.m_total && g.image_out) {
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {  // bf16 +1 = 0x3f80 where d < 0, -1 = 0xbf80 otherwise: only the sign bit differs
                const uint32_t hi = __byte_perm(__float_as_uint(d[2 * j]), __float_as_uint(d[2 * j + 1]), 0x7632);  // high halves of both
                w[j] = (hi & 0x80008000u) ^ 0xbf80bf80u;
            }
            uint4* dst = reinterpret_cast<uint4*>(g.image_out + static_cast<int64_t>(row) * g.image_pitch + col0);
            if (col0 + 16 <= g.image_pitch) {
                dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
        }
    } else if (EPI == EPI_FIELDS) {
        // row = chain, columns = nodes: the field exactly as the sampling epilogue forms it (bias + f32 accumulator)
        if (row < g.m_total) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (col0 + j < g.n_total)
                    g.fields_out[static_cast<int64_t>(row) * g.n_total + col0 + j] = __fadd_rn(__ldg(g.bias + col0 + j), __uint_as_float(acc[j]));
        }
    } else {
        // row = node of block a, columns = nodes of block b; acc = N11 (int32)
        if (row < g.m_total) {
            const int32_t na = __ldg(g.ones_a + row);
            float out[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int col = col0 + j;
                const int32_t nb = col < g.n_total ? __ldg(g.ones_b + col) : 0;
                const int32_t sum = 4 * static_cast<int32_t>(acc[j]) - 2 * na - 2 * nb + g.n_chains;
                out[j] = __fdiv_rn(static_cast<float>(sum), static_cast<float>(g.n_chains));
            }
            float* dst = g.corr_out + static_cast<int64_t>(row) * g.n_total + col0;
            if (g.corr_transposed) {  // the caller swapped the operands: write out[col][row]; a warp's 32 rows are contiguous
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (col0 + j < g.n_total) g.corr_out[static_cast<int64_t>(col0 + j) * g.m_total + row] = out[j];
            } else if (col0 + 16 <= g.n_total && (g.n_total & 3) == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) reinterpret_cast<float4*>(dst)[j] = make_float4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (col0 + j < g.n_total) dst[j] = out[j];
            }
        }
    }
}

template <int BN>
__host__ __device__ constexpr int stages_for() { return STAGE_BUDGET / ((BM + BN) * BK_BYTES); }

template <int EPI, int BN>
__global__ void __launch_bounds__(THREADS, 1) k_dense_gemm(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                           const __grid_constant__ GemmArgs g) {
    constexpr int KIND_I8 = EPI == EPI_CORR;
    constexpr int STAGES = stages_for<BN>();
    constexpr uint32_t A_BYTES = BM * BK_BYTES, B_BYTES = BN * BK_BYTES, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t TMEM_COLS = ACC_BUFS * BN;  // 128 or 256: a power of two >= 32
    constexpr uint32_t IDESC = KIND_I8 ? make_idesc(2, 0, BM, BN) : make_idesc(1, 1, BM, BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[ACC_BUFS], acc_empty[ACC_BUFS];
    __shared__ uint32_t tmem_base_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = g.tiles_m * g.tiles_n;
    const int k_tiles = (g.k_bytes + BK_BYTES - 1) / BK_BYTES;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < ACC_BUFS; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ---- TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
                const int tm = tile / g.tiles_n, tn = tile % g.tiles_n;
                for (int kt = 0; kt < k_tiles; ++kt) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, g.err, 1)) { alive = false; break; }
                    mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
                    const uint32_t dst = smem_u32(smem + stage * STAGE_BYTES);
                    const int32_t kx = kt * (BK_BYTES / (KIND_I8 ? 1 : 2));  // tensor-map coordinates count elements
                    tma_load_2d(dst, &map_a, &full_bar[stage], kx, tm * BM);
                    tma_load_2d(dst + A_BYTES, &map_b, &full_bar[stage], kx, tn * BN);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, it = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++it) {
                const uint32_t buf = it & 1u, use = it >> 1;
                if (!mbar_wait(&acc_empty[buf], (use & 1u) ^ 1u, g.err, 2)) { alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + buf * BN;
                for (int kt = 0; kt < k_tiles; ++kt) {
                    if (!mbar_wait(&full_bar[stage], phase, g.err, 3)) { alive = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
                    const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int ks = 0; ks < BK_BYTES / 32; ++ks)  // one MMA consumes 32 bytes of K (16 bf16 or 32 int8)
                        umma<KIND_I8>(tmem_d, da + static_cast<uint64_t>(ks * 2), db + static_cast<uint64_t>(ks * 2), IDESC, (kt | ks) ? 1u : 0u);
                    umma_commit(&empty_bar[stage]);  // frees the stage when these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (alive) umma_commit(&acc_full[buf]);
            }
        }
    } else {
        // ---- epilogue warps
        const int quarter = warp & 3;         // TMEM lanes [32*quarter, 32*quarter+32)
        const int col_group = (warp - 2) >> 2;  // which quarter of the tile's 16-column chunks this warp finishes
        uint32_t it = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x, ++it) {
            const int tm = tile / g.tiles_n, tn = tile % g.tiles_n;
            const uint32_t buf = it & 1u, use = it >> 1;
            if (!mbar_wait(&acc_full[buf], use & 1u, g.err, 4)) { alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int c = col_group; c < BN / 16; c += EPI_WARPS / 4) {
                uint32_t acc[16];
                tmem_ld16_issue(taddr + c * 16, acc);
                tmem_ld_wait();
                finish_chunk<EPI>(g, acc, tm * BM + quarter * 32, tn * BN + c * 16, lane);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster (two SMs) share one 256 x BN output tile through tcgen05 cta_group::2.
// Each CTA stages its own 128 rows of A and only HALF of the B tile (BN/2 rows); the tensor cores of both SMs read
// both halves, so the B operand crosses the L2-to-SM fabric once per pair instead of once per CTA.  The update GEMMs
// here are bound by that operand feed, not by the tensor pipe.
// Roles per CTA as in k_dense_gemm.  Hand-overs: every TMA load of either CTA completes on the LEADER's (rank 0) full
// barrier; the leader's single MMA thread issues the pair's MMAs and commits each stage to the empty barrier of both
// CTAs and each finished accumulator to the full barrier of both; the epilogue warps of both CTAs release an
// accumulator on the leader's barrier.  Every load and every arrival names one destination CTA.  All waits are bounded; a cluster barrier
// before exit keeps either CTA's shared memory alive until its peer's last remote arrival.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory object in the CTA of the given cluster rank.
__device__ __forceinline__ uint32_t peer_addr(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion is counted on a barrier that may live in the pair's other CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
                 : "memory");
}
template <int KIND_I8>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if (KIND_I8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
// Arrival (once the pair's earlier MMAs have completed) on a barrier given by its cluster address.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

constexpr int PAIR_BM = 256;  // rows of the pair's tile: 128 per CTA
template <int BN>
__host__ __device__ constexpr int pair_stages_for() { return STAGE_BUDGET / ((BM + BN / 2) * BK_BYTES); }

template <int EPI, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
    k_dense_gemm_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ GemmArgs g) {
    static_assert(BN % 16 == 0 && BN >= 32 && BN <= 256, "pair tile width");
    constexpr int KIND_I8 = EPI == EPI_CORR;
    constexpr int BH = BN / 2;  // rows of B this CTA stages
    constexpr int STAGES = pair_stages_for<BN>();
    constexpr uint32_t A_BYTES = BM * BK_BYTES, B_BYTES = BH * BK_BYTES, STAGE_BYTES = A_BYTES + B_BYTES;
    static_assert(B_BYTES % 1024 == 0, "each stage starts on a swizzle-atom boundary");
    constexpr uint32_t ACC_STRIDE = BN > 128 ? 256 : 128;  // TMEM columns between the two accumulators
    constexpr uint32_t TMEM_COLS = ACC_BUFS * ACC_STRIDE;
    constexpr uint32_t IDESC = KIND_I8 ? make_idesc(2, 0, PAIR_BM, BN) : make_idesc(1, 1, PAIR_BM, BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[ACC_BUFS], acc_empty[ACC_BUFS];
    __shared__ uint32_t tmem_base_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const int n_tiles = g.tiles_m * g.tiles_n;
    const int k_tiles = (g.k_bytes + BK_BYTES - 1) / BK_BYTES;
    const int first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < ACC_BUFS; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // one warp of each CTA of the pair takes part in the allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();  // barriers of both CTAs initialised and TMEM allocated before anything crosses the pair
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;
    if (g.debug && threadIdx.x == 0) g.debug[blockIdx.x & 1] = tmem_base;

    if (warp == 0) {
        // ---- TMA producer (both CTAs); completion is counted on the leader's barrier
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool alive = true;
            for (int tile = first_tile; tile < n_tiles && alive; tile += tile_step) {
                const int tm = tile / g.tiles_n, tn = tile % g.tiles_n;
                for (int kt = 0; kt < k_tiles; ++kt) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, g.err, 1)) { alive = false; break; }
                    if (leader) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
                    const uint32_t bar = peer_addr(smem_u32(&full_bar[stage]), 0);
                    const uint32_t dst = smem_u32(smem + stage * STAGE_BYTES);
                    const int32_t kx = kt * (BK_BYTES / (KIND_I8 ? 1 : 2));
                    tma_load_2d_pair(dst, &map_a, bar, kx, tm * PAIR_BM + static_cast<int32_t>(rank) * BM);
                    tma_load_2d_pair(dst + A_BYTES, &map_b, bar, kx, tn * BN + static_cast<int32_t>(rank) * BH);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: the leader's thread drives the tensor cores of both SMs
        if (lane == 0 && leader) {
            uint32_t stage = 0, phase = 0, it = 0;
            bool alive = true;
            for (int tile = first_tile; tile < n_tiles && alive; tile += tile_step, ++it) {
                const uint32_t buf = it & 1u, use = it >> 1;
                if (!mbar_wait(&acc_empty[buf], (use & 1u) ^ 1u, g.err, 2)) { alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + buf * ACC_STRIDE;
                for (int kt = 0; kt < k_tiles; ++kt) {
                    if (!mbar_wait(&full_bar[stage], phase, g.err, 3)) { alive = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(smem + stage * STAGE_BYTES);
                    const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int ks = 0; ks < BK_BYTES / 32; ++ks)
                        umma_pair<KIND_I8>(tmem_d, da + static_cast<uint64_t>(ks * 2), db + static_cast<uint64_t>(ks * 2), IDESC, (kt | ks) ? 1u : 0u);
                    const uint32_t e = smem_u32(&empty_bar[stage]);
                    umma_commit_pair(e);                // frees the stage here ...
                    umma_commit_pair(peer_addr(e, 1));  // ... and in the peer
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (alive) {
                    const uint32_t f = smem_u32(&acc_full[buf]);
                    umma_commit_pair(f);
                    umma_commit_pair(peer_addr(f, 1));
                }
            }
        }
    } else {
        // ---- epilogue warps: each CTA finishes its own 128 rows of the pair's tile
        const int quarter = warp & 3;
        const int col_group = (warp - 2) >> 2;
        uint32_t it = 0;
        bool alive = true;
        for (int tile = first_tile; tile < n_tiles && alive; tile += tile_step, ++it) {
            const int tm = tile / g.tiles_n, tn = tile % g.tiles_n;
            const uint32_t buf = it & 1u, use = it >> 1;
            if (!mbar_wait(&acc_full[buf], use & 1u, g.err, 4)) { alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + buf * ACC_STRIDE + (static_cast<uint32_t>(quarter * 32) << 16);
            const int row_base = tm * PAIR_BM + static_cast<int>(rank) * BM + quarter * 32;
#pragma unroll 1
            for (int c = col_group; c < BN / 16; c += EPI_WARPS / 4) {
                uint32_t acc[16];
                tmem_ld16_issue(taddr + c * 16, acc);
                tmem_ld_wait();
                finish_chunk<EPI>(g, acc, row_base, tn * BN + c * 16, lane);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(peer_addr(smem_u32(&acc_empty[buf]), 0));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();  // no CTA leaves (or frees TMEM) while its peer can still reach it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// 0/1 byte state [node][chain] of one block -> +-1 bf16 image [chain][node] (columns from n up to the pitch are zero)
// and, when `ones` is given, the number of ones per node over the existing chains, added with atomics (the caller
// zeroes it).  A CTA moves a tile of 32 nodes x 128 chains: 128-byte row segments in, 64-byte image segments out.
__global__ void __launch_bounds__(256) k_make_image(const uint8_t* rows, int64_t ld, int64_t n_chains, int32_t n, __nv_bfloat16* image, int64_t pitch, int32_t* ones) {
    __shared__ uint32_t tile[32][33];  // [node][word of four chains]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t node0 = static_cast<int64_t>(blockIdx.x) * 32, chain0 = static_cast<int64_t>(blockIdx.y) * 128;
    for (int r = warp; r < 32; r += 8) {
        const int64_t node = node0 + r, chain = chain0 + 4 * lane;
        uint32_t w = 0;
        if (node < n && chain < n_chains) {  // ld is a multiple of 16, so a word that starts below n_chains lies inside the row
            w = *reinterpret_cast<const uint32_t*>(rows + node * ld + chain);
            const int64_t left = n_chains - chain;
            if (left < 4) w &= 0xffffffffu >> (8 * (4 - static_cast<int>(left)));
        }
        tile[r][lane] = w;
        if (ones) {
            const int cnt = __reduce_add_sync(0xffffffffu, __popc(w & 0x01010101u));
            if (lane == 0 && cnt) atomicAdd(ones + node, cnt);
        }
    }
    __syncthreads();
    const int c = threadIdx.x >> 1, h = threadIdx.x & 1;  // chain of the tile, which 16 of the 32 nodes
    const int64_t chain = chain0 + c;
    if (chain < n_chains && node0 + 16 * h + 16 <= pitch) {
        uint32_t out[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int r0 = 16 * h + 2 * j;
            const uint32_t b0 = (tile[r0][c >> 2] >> (8 * (c & 3))) & 1u, b1 = (tile[r0 + 1][c >> 2] >> (8 * (c & 3))) & 1u;
            const uint32_t v0 = node0 + r0 < n ? (b0 ? 0x3f80u : 0xbf80u) : 0u, v1 = node0 + r0 + 1 < n ? (b1 ? 0x3f80u : 0xbf80u) : 0u;  // bf16 +1 / -1
            out[j] = v0 | (v1 << 16);
        }
        uint4* dst = reinterpret_cast<uint4*>(image + chain * pitch + node0 + 16 * h);
        dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
        dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
    }
}
// Number of ones per state row (over existing chains).
__global__ void k_row_ones(const uint8_t* rows, int64_t ld, int64_t n_chains, int32_t n, int32_t* out) {
    const int64_t node = static_cast<int64_t>(blockIdx.x) * 8 + threadIdx.y;
    if (node >= n) return;
    int cnt = 0;
    for (int64_t quad = threadIdx.x; 4 * quad < n_chains; quad += 32) {
        uint32_t wd = *reinterpret_cast<const uint32_t*>(rows + node * ld + 4 * quad);
        const int64_t left = n_chains - 4 * quad;
        if (left < 4) wd &= 0xffffffffu >> (8 * (4 - static_cast<int>(left)));
        cnt += __popc(wd & 0x01010101u);
    }
    cnt = __reduce_add_sync(0xffffffffu, cnt);
    if (threadIdx.x == 0) out[node] = cnt;
}

}  // namespace dense
}  // namespace thrml
