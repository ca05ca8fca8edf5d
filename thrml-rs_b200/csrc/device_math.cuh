// Counter-based noise and deterministic f32 math used inside the kernels.
//
// The reference never consumes its RngKey (every sampler draws from Burn's global generator), so the mapping from a
// block's key to the noise of each (node, chain) is this engine's own definition:
//   Philox4x32-10, key = (low, high) 32 bits of the block's RngKey, counter = (node index inside the block,
//   chain word, lane, tag).  A spin update of global chain c uses output word c&3 of counter (node, c>>2, 0, TAG_SPIN);
//   category k of a categorical update uses word k&3 of counter (node, c, k>>2, TAG_CAT).
// exp/sigmoid/log are fixed sequences of IEEE-754 single-precision operations (no MUFU approximations, no fused
// contraction beyond the fmaf calls written out), so a CPU evaluating the same sequence gets the same bits.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace thrml {

constexpr uint32_t TAG_SPIN = 0x5350494Eu;
constexpr uint32_t TAG_CAT = 0x43415447u;
constexpr uint32_t TAG_HINT = 0x48494E54u;
constexpr uint32_t TAG_RAND = 0x52414E44u;

struct U4 {
    uint32_t x, y, z, w;
};

__device__ __forceinline__ U4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0, p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;  // one wide multiply each
        const uint32_t hi0 = static_cast<uint32_t>(p0 >> 32), lo0 = static_cast<uint32_t>(p0);
        const uint32_t hi1 = static_cast<uint32_t>(p1 >> 32), lo1 = static_cast<uint32_t>(p1);
        c0 = hi1 ^ c1 ^ k0;
        c1 = lo1;
        c2 = hi0 ^ c3 ^ k1;
        c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return U4{c0, c1, c2, c3};
}

// The same function with the ten round keys (key + r * Weyl constant) supplied by the caller: kernels whose block key is
// a launch parameter keep them in the parameter (constant) bank, which removes two integer adds per round.
struct PhiloxRoundKeys {
    uint32_t k0[10], k1[10];
};
inline PhiloxRoundKeys make_round_keys(uint64_t key) {
    PhiloxRoundKeys rk;
    for (int r = 0; r < 10; ++r) {
        rk.k0[r] = static_cast<uint32_t>(key) + static_cast<uint32_t>(r) * 0x9E3779B9u;
        rk.k1[r] = static_cast<uint32_t>(key >> 32) + static_cast<uint32_t>(r) * 0xBB67AE85u;
    }
    return rk;
}
__device__ __forceinline__ U4 philox4x32_10_rk(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, const PhiloxRoundKeys& rk) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0, p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;  // one wide multiply each
        const uint32_t hi0 = static_cast<uint32_t>(p0 >> 32), lo0 = static_cast<uint32_t>(p0);
        const uint32_t hi1 = static_cast<uint32_t>(p1 >> 32), lo1 = static_cast<uint32_t>(p1);
        c0 = hi1 ^ c1 ^ rk.k0[r];
        c1 = lo1;
        c2 = hi0 ^ c3 ^ rk.k1[r];
        c3 = lo0;
    }
    return U4{c0, c1, c2, c3};
}

__device__ __forceinline__ uint32_t pick(const U4& v, uint32_t i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }

// Hardware base-2 logarithm for normal positive inputs (the screens of the Gumbel draws: u >= 2^-24 and -ln u >= 2^-24).  The
// flush-to-zero form is one instruction; the default form adds a range test and a rescaling for subnormal inputs that
// cannot occur here.
__device__ __forceinline__ float lg2_normal(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Hardware reciprocal for normal inputs, one instruction.
__device__ __forceinline__ float rcp_normal(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 24-bit uniform in [0,1) and 23-bit uniform strictly inside (0,1).
__device__ __forceinline__ float u24(uint32_t r) { return __fmul_rn(__uint2float_rn(r >> 8), 5.9604644775390625e-8f); }
__device__ __forceinline__ float u23_open(uint32_t r) {
    return __fmul_rn(__fadd_rn(__uint2float_rn(r >> 9), 0.5f), 1.1920928955078125e-7f);
}

// exp(t) for t <= 0 (0 below -86).
__device__ __forceinline__ float det_exp_nonpos(float t) {
    if (t < -86.0f) return 0.0f;
    const float n = rintf(__fmul_rn(t, 1.44269504088896341f));
    float r = __fmaf_rn(n, -0.693359375f, t);
    r = __fmaf_rn(n, 2.12194440e-4f, r);
    const float z = __fmul_rn(r, r);
    float y = 1.9875691500e-4f;
    y = __fmaf_rn(y, r, 1.3981999507e-3f);
    y = __fmaf_rn(y, r, 8.3334519073e-3f);
    y = __fmaf_rn(y, r, 4.1665795894e-2f);
    y = __fmaf_rn(y, r, 1.6666665459e-1f);
    y = __fmaf_rn(y, r, 5.0000001201e-1f);
    y = __fmaf_rn(y, z, r);
    y = __fadd_rn(y, 1.0f);
    const int32_t e = static_cast<int32_t>(n) + 127;
    return __fmul_rn(y, __uint_as_float(static_cast<uint32_t>(e) << 23));
}
// 1/(1+exp(-x)), evaluated on the side that cannot overflow.
__device__ __forceinline__ float det_sigmoid(float x) {
    if (x >= 0.0f) {
        const float e = det_exp_nonpos(-x);
        return __fdiv_rn(1.0f, __fadd_rn(1.0f, e));
    }
    const float e = det_exp_nonpos(x);
    return __fdiv_rn(e, __fadd_rn(1.0f, e));
}
// ln(x) for positive normal x.
__device__ __forceinline__ float det_log(float x) {
    uint32_t bits = __float_as_uint(x);
    int32_t e = static_cast<int32_t>((bits >> 23) & 0xffu) - 126;
    float m = __uint_as_float((bits & 0x007fffffu) | 0x3f000000u);
    if (m < 0.707106781186547524f) {
        e -= 1;
        m = __fadd_rn(m, m);
    }
    const float f = __fadd_rn(m, -1.0f);
    const float z = __fmul_rn(f, f);
    float y = 7.0376836292e-2f;
    y = __fmaf_rn(y, f, -1.1514610310e-1f);
    y = __fmaf_rn(y, f, 1.1676998740e-1f);
    y = __fmaf_rn(y, f, -1.2420140846e-1f);
    y = __fmaf_rn(y, f, 1.4249322787e-1f);
    y = __fmaf_rn(y, f, -1.6668057665e-1f);
    y = __fmaf_rn(y, f, 2.0000714765e-1f);
    y = __fmaf_rn(y, f, -2.4999993993e-1f);
    y = __fmaf_rn(y, f, 3.3333331174e-1f);
    y = __fmul_rn(y, f);
    y = __fmul_rn(y, z);
    const float fe = static_cast<float>(e);
    y = __fmaf_rn(fe, -2.12194440e-4f, y);
    y = __fmaf_rn(z, -0.5f, y);
    float r = __fadd_rn(f, y);
    r = __fmaf_rn(fe, 0.693359375f, r);
    return r;
}

}  // namespace thrml
