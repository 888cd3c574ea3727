// quantize_e8mx (ref: 1243-1428): keep the 8-bit exponent, round the mantissa to M bits, under an optional
// tensor-wide scale.  Shared by the streaming kernel (fq_elementwise.cu) and the single-launch kernel for small
// tensors (fq_resident.cu).
#pragma once

#include "kernels.cuh"

namespace morb {
namespace {

// ref: 1243-1327: keep the exponent, round the mantissa to M bits.  The reference's
// threshold ladder is round-to-nearest-even on the top seven mantissa bits: index j
// is kept while man <= j*step + step/2 (even j) or that minus 65536 (odd j).
template <int M>
__device__ __forceinline__ float e8m_round(float v) {
    const uint32_t b = f2u(v);
    uint32_t e = (b >> 23) & 0xFFu, man = b & 0x7FFFFFu;
    if (e == 0) man = 0;
    else if (e != 255) {
        constexpr uint32_t step = 0x800000u >> M;
        constexpr uint32_t steps = 1u << M;
        uint32_t k = steps;
#pragma unroll
        for (int j = (int)steps - 1; j >= 0; --j) {
            const uint32_t lim = (uint32_t)j * step + step / 2 - ((j & 1) ? 65536u : 0u);
            if (man <= lim) k = (uint32_t)j;
        }
        if (k < steps) man = k * step;
        else {
            man = 0;
            e += 1;
            if (e == 255) { e = 254; man = (steps - 1) * step; }
        }
    }
    return u2f((b & 0x80000000u) | (e << 23) | man);
}

// ref: 1335-1359
template <int M>
__device__ __forceinline__ float e8mx_scale(float gamax, int strategy) {
    if (strategy != 1) return 1.0f;
    const uint32_t e = (f2u(gamax) >> 23) + 1;
    const float fp_max = u2f((e << 23) | (((1u << M) - 1u) << (23 - M)));
    float s = __fdiv_rn(fp_max, gamax);
    if (s >= 2.0f) s = __fdiv_rn(s, 2.0f);
    return s;
}

// One CTA's view of the cast.  Every step of `one` commutes with a power of two as long as nothing leaves the
// normal range (the product and the quotient are correctly rounded, the mantissa rounding keeps the exponent or
// raises it by one), and the result has the sign of the input: for an exponent field in [2, 251] the output
// pattern is the input pattern plus a small offset that depends on the seven mantissa bits only.  The 128
// offsets are tabulated per CTA with the literal arithmetic; zeros give +0 as in the reference; anything else
// (subnormals, the top binades, Inf, NaN) takes the literal path.
template <int M>
struct E8mxCast {
    const uint32_t* off;   // 128 entries in shared memory: offset + 256, so that the packed sum below never borrows
    float s;
    __device__ __forceinline__ float one(float x) const {
        const float v = __fmul_rn(x, s);
        float d = 0.0f;
        if (v != 0.0f) d = e8m_round<M>(v);
        return __fdiv_rn(d, s);
    }
    // threads 0..127 fill the table; the caller synchronises the CTA before the first word()
    __device__ __forceinline__ void init(uint32_t* table, float scale, int tid) {
        off = table;
        s = scale;
        if (tid < 128) {
            const uint32_t pat = (127u << 7) | (uint32_t)tid;
            table[tid] = f32_to_bf16_bits(one(u2f(pat << 16))) + 256u - pat;
        }
    }
    __device__ __forceinline__ uint32_t slow_word(uint32_t w) const { return pack_bf16(one(bf16_hi(w)), one(bf16_lo(w))); }
    __device__ __forceinline__ uint32_t word(uint32_t w) const {
        const uint32_t m = mag2(w);
        const uint32_t nz = (((m + 0x7FFF7FFFu) & 0x80008000u) >> 15) * 0xFFFFu;   // 0xFFFF in every non-zero half
        const uint32_t mp = m | (~nz & 0x3F803F80u);                               // a zero half stands in as 1.0
        if (umax16x2(mp, 0x01000100u) != mp || umin16x2(mp, 0x7DFF7DFFu) != mp) return slow_word(w);
        const uint32_t o = off[mp & 0x7Fu] + (off[(mp >> 16) & 0x7Fu] << 16);
        return ((mp + o - 0x01000100u) | (w & 0x80008000u)) & nz;
    }
};

}  // namespace
}  // namespace morb
