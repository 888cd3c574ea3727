// Device-side building blocks shared by every kernel of libmor_b200 (sm_100a only).
//
// All arithmetic is IEEE binary32 with explicit rounding intrinsics (__fmul_rn,
// __fdiv_rn, __fadd_rn) so that nvcc can neither contract nor reorder it; the
// results must match, bit for bit, the arithmetic of the reference operators in
// mor/csrc/cuda/fake_quantize.cu of boryiings/mor ("ref:" line numbers below).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace morb {

// ----------------------------------------------------------------------------
// status codes of the C-ABI (include/mor_b200.h)
// ----------------------------------------------------------------------------
constexpr int kOk = 0;
constexpr int kErrInvalidArgument = -1;
constexpr int kErrUnsupportedShape = -2;
constexpr int kErrWorkspace = -3;
constexpr int kErrLaunch = -4;
constexpr int kErrTooLarge = -5;

// narrow formats
enum Fmt : int { kE4M3 = 0, kE5M2 = 1, kE3M2 = 2, kE2M3 = 3 };
// scale kinds (ref: 62-65)
enum Sf : int { kSfFp32 = 1, kSfE8 = 2 };

__device__ __forceinline__ uint32_t f2u(float f) { return __float_as_uint(f); }
__device__ __forceinline__ float u2f(uint32_t u) { return __uint_as_float(u); }

// A packed word holds element 2w in its low half and element 2w+1 in its high half.
__device__ __forceinline__ float bf16_lo(uint32_t w) { return u2f(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return u2f(w & 0xFFFF0000u); }

// ref: 46-60.  Round half away from zero on bit 15; the reference ORs the exponent
// field over the sign, so a NaN whose top eight mantissa bits are ones becomes
// 0x8000 whatever its sign.
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float v) {
    const uint32_t b = f2u(v);
    uint32_t r = (b + 0x8000u) >> 16;
    if ((b & 0x7FFF8000u) == 0x7FFF8000u) r = 0x8000u;
    return r;
}
__device__ __forceinline__ uint32_t pack_bf16(float hi, float lo) {
    return (f32_to_bf16_bits(hi) << 16) | f32_to_bf16_bits(lo);
}

// ----------------------------------------------------------------------------
// hardware narrow-float conversions (PTX ISA 8.6+, sm_100a)
// ----------------------------------------------------------------------------
// Two binary32 values -> two codes, RNE, saturate-to-finite, NaN -> NaN code.
// Upper byte = code of `hi`, lower byte = code of `lo`.
template <int FMT>
__device__ __forceinline__ uint32_t cvt_codes(float hi, float lo) {
    uint16_t r;
    if constexpr (FMT == kE4M3) asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    else if constexpr (FMT == kE5M2) asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    else if constexpr (FMT == kE2M3) asm("cvt.rn.satfinite.e2m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    else asm("cvt.rn.satfinite.e3m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
// Two codes -> half2 bits (exact).
template <int FMT>
__device__ __forceinline__ uint32_t codes_to_h2(uint32_t codes) {
    uint32_t r;
    const uint16_t c = (uint16_t)codes;
    if constexpr (FMT == kE4M3) asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(c));
    else if constexpr (FMT == kE5M2) asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(r) : "h"(c));
    else if constexpr (FMT == kE2M3) asm("cvt.rn.f16x2.e2m3x2 %0, %1;" : "=r"(r) : "h"(c));
    else asm("cvt.rn.f16x2.e3m2x2 %0, %1;" : "=r"(r) : "h"(c));
    return r;
}
__device__ __forceinline__ float h_lo_to_f32(uint32_t h2) { return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu))); }
__device__ __forceinline__ float h_hi_to_f32(uint32_t h2) { return __half2float(__ushort_as_half((unsigned short)(h2 >> 16))); }

// ref: 218-245 with T_USE_CUDA_CAST = true for E4M3/E5M2 (static_cast through
// __nv_fp8_e4m3/e5m2: RNE, saturate-to-finite, zero keeps its sign) and the custom
// cast for E2M3 (ref: 125-215: same grid and rounding, but a zero result is +0).
template <int FMT, bool FINITE = false>
__device__ __forceinline__ void quant_dequant_pair(float hi, float lo, float& qhi, float& qlo) {
    uint32_t h2 = codes_to_h2<FMT>(cvt_codes<FMT>(hi, lo));
    if constexpr (FMT == kE2M3 || FMT == kE3M2) {
        // -0 -> +0 on both halves at once: bit 15 of (|h| + 0x7FFF) is set iff the half is non-zero
        const uint32_t nz = ((h2 & 0x7FFF7FFFu) + 0x7FFF7FFFu) & 0x80008000u;
        h2 &= nz | 0x7FFF7FFFu;
    }
    qhi = h_hi_to_f32(h2);
    qlo = h_lo_to_f32(h2);
    if constexpr ((FMT == kE2M3 || FMT == kE3M2) && !FINITE) {
        // no NaN encoding: the custom cast clamps NaN/Inf to the signed maximum,
        // the hardware returns +max for NaN.
        if (hi != hi) qhi = copysignf(qhi, hi);
        if (lo != lo) qlo = copysignf(qlo, lo);
    }
}

// ----------------------------------------------------------------------------
// the custom cast of the test operators (ref: 125-215), integer formulation
// ----------------------------------------------------------------------------
template <int EBITS, int MBITS, int BIAS, int TOP, bool SATURATES, bool E4M3_NAN>
__device__ __forceinline__ float narrow_custom(float x) {
    const uint32_t b = f2u(x);
    const uint32_t sign = b & 0x80000000u;
    constexpr int drop = 23 - MBITS;
    constexpr uint32_t mmask = (1u << MBITS) - 1u;
    int e = (int)((b >> 23) & 0xFFu) - 127 + BIAS;
    uint32_t man = 0, guard = 0, sticky = 0;
    if (e > 0) {
        man = (b >> drop) & mmask;
        guard = (b >> (drop - 1)) & 1u;
        sticky = (b & ((1u << (drop - 1)) - 1u)) != 0;
    } else {
        const int rs = 1 - e;
        e = 0;
        if (rs <= MBITS + 1) {
            uint32_t sig = (b & 0x7FFFFFu) | (1u << 23);
            sticky = (sig & ((1u << (rs + drop - 1)) - 1u)) != 0;
            sig >>= rs;
            guard = (sig >> (drop - 1)) & 1u;
            man = (sig >> drop) & mmask;
        }
    }
    if (guard && (sticky || (man & 1u))) {
        man += 1;
        if (man == (1u << MBITS)) { man = 0; e += 1; }
    }
    if constexpr (SATURATES) {
        if (e > TOP) { e = (1 << EBITS) - 1; man = mmask; }
    } else {
        if (e > TOP) return u2f(0x7FFFFFFFu);
        if (E4M3_NAN && e == TOP && man == mmask) return u2f(0x7FFFFFFFu);
    }
    uint32_t out = 0;
    if (e > 0) {
        out = sign | ((uint32_t)(e + 127 - BIAS) << 23) | (man << drop);
    } else if (man) {
        const int lead = 31 - __clz((int)man);          // position of the leading one, < MBITS
        const int ex = 127 - BIAS + 1 - (MBITS - lead);  // each left shift lowers the exponent
        man = (man << (MBITS - lead)) & mmask;
        out = sign | ((uint32_t)ex << 23) | (man << drop);
    }
    return u2f(out);
}
template <int FMT>
__device__ __forceinline__ float narrow_custom_fmt(float x) {
    if constexpr (FMT == kE4M3) return narrow_custom<4, 3, 7, 15, false, true>(x);
    else if constexpr (FMT == kE5M2) return narrow_custom<5, 2, 15, 30, false, false>(x);
    else if constexpr (FMT == kE3M2) return narrow_custom<3, 2, 3, 7, true, false>(x);
    else return narrow_custom<2, 3, 1, 3, true, false>(x);
}

// ----------------------------------------------------------------------------
// scale, quantize, dequantize, descale
// ----------------------------------------------------------------------------
// ref: 248-306 with E8_RZ: power-of-two scale applied to the exponent FIELD.
// e8 = exponent field of the scale - 127.  The field is clamped at 0 on the way in
// and on the way out and the mantissa rides along, so zeros and subnormals are not
// special: with e8 < 0 a value that quantizes to 0 comes back as 2^(-e8-127).
__device__ __forceinline__ int e8_of_scale(float s) { return (int)((f2u(s) >> 23) & 0xFFu) - 127; }

__device__ __forceinline__ float e8_shift_field(float v, int delta) {
    const uint32_t b = f2u(v);
    int t = (int)(b & 0x7FFFFFFFu) + delta * (1 << 23);
    // a negative field keeps only the mantissa; the low 23 bits are untouched by the add
    t &= ~((t >> 31) & (int)0xFF800000);
    return u2f((b & 0x80000000u) | (uint32_t)t);
}

template <int FMT>
__device__ __forceinline__ void sqdd_e8_pair(float hi, float lo, int e8, float& rhi, float& rlo) {
    float qhi, qlo;
    quant_dequant_pair<FMT>(e8_shift_field(hi, e8), e8_shift_field(lo, e8), qhi, qlo);
    rhi = e8_shift_field(qhi, -e8);
    rlo = e8_shift_field(qlo, -e8);
}

// ref: 310-316: multiply, cast, TRUE division (not a reciprocal multiply).
template <int FMT>
__device__ __forceinline__ void sqdd_fp32_pair(float hi, float lo, float s, float& rhi, float& rlo) {
    float qhi, qlo;
    quant_dequant_pair<FMT>(__fmul_rn(hi, s), __fmul_rn(lo, s), qhi, qlo);
    rhi = __fdiv_rn(qhi, s);
    rlo = __fdiv_rn(qlo, s);
}

template <int FMT, int SF>
__device__ __forceinline__ void sqdd_pair(float hi, float lo, float s, float& rhi, float& rlo) {
    if constexpr (SF == kSfE8) sqdd_e8_pair<FMT>(hi, lo, e8_of_scale(s), rhi, rlo);
    else sqdd_fp32_pair<FMT>(hi, lo, s, rhi, rlo);
}

// ----------------------------------------------------------------------------
// fast forms, bit-identical to the ones above on their stated domains
// ----------------------------------------------------------------------------
// 2^e as a float, -126 <= e <= 127
__device__ __forceinline__ float pow2f(int e) { return u2f((uint32_t)(e + 127) << 23); }

// Two floats -> packed bf16 word with the reference's round-half-away rule.  Exact
// for every input except a NEGATIVE NaN whose top eight mantissa bits are ones (the
// reference maps that to 0x8000, the plain add wraps to 0); callers canonicalise NaNs
// to +0x7fffffff, for which the add gives 0x8000 as required.
__device__ __forceinline__ uint32_t pack_bf16_round(float hi, float lo) {
    return __byte_perm(f2u(lo) + 0x8000u, f2u(hi) + 0x8000u, 0x7632);
}
// Two floats whose low 16 bits are zero (results of the power-of-two path) -> packed word
__device__ __forceinline__ uint32_t pack_bf16_trunc(float hi, float lo) {
    return __byte_perm(f2u(lo), f2u(hi), 0x7632);
}
__device__ __forceinline__ float canon_nan(float v) { return (v != v) ? u2f(0x7FFFFFFFu) : v; }

// Power-of-two (E8) scaling as two float multiplies instead of exponent-field
// arithmetic.  For -119 <= e8 <= 100 and finite x the field arithmetic of the
// reference (ref: 283-305) and x * 2^e8 give the same narrow-float code: both scale a
// normal value exactly, and whatever lands below 2^-126 casts to a signed zero either
// way; on the way back q * 2^-e8 is exact for every non-zero code.  The one
// difference is a code of zero with e8 < 0: the field arithmetic returns
// +-2^(-e8-127), restored here with a select.  e8 outside the range takes the literal
// path.
__device__ __forceinline__ bool e8_fast_ok(int e8) { return e8 >= -119 && e8 <= 100; }

template <int FMT>
__device__ __forceinline__ void sqdd_e8_pair_fast(float hi, float lo, float up, float down, uint32_t zero_bits,
                                                  float& rhi, float& rlo) {
    float qhi, qlo;
    quant_dequant_pair<FMT>(__fmul_rn(hi, up), __fmul_rn(lo, up), qhi, qlo);
    rhi = __fmul_rn(qhi, down);
    rlo = __fmul_rn(qlo, down);
    if (zero_bits) {  // e8 < 0: a zero code comes back as 2^(-e8-127) with the sign of the code
        if (qhi == 0.0f) rhi = u2f((f2u(qhi) & 0x80000000u) | zero_bits);
        if (qlo == 0.0f) rlo = u2f((f2u(qlo) & 0x80000000u) | zero_bits);
    }
}
struct E8Consts {
    float up, down;        // 2^e8, 2^-e8
    uint32_t zero_bits;    // (-e8) << 23 when e8 < 0, else 0
    int e8;
    bool fast;
};
__device__ __forceinline__ E8Consts e8_consts(float scale) {
    E8Consts c;
    c.e8 = e8_of_scale(scale);
    c.fast = e8_fast_ok(c.e8);
    const int e = c.fast ? c.e8 : 0;
    c.up = pow2f(e);
    c.down = pow2f(-e);
    c.zero_bits = e < 0 ? ((uint32_t)(-e) << 23) : 0u;
    return c;
}
template <int FMT>
__device__ __forceinline__ void sqdd_e8_pair_auto(float hi, float lo, const E8Consts& c, float& rhi, float& rlo) {
    if (c.fast) sqdd_e8_pair_fast<FMT>(hi, lo, c.up, c.down, c.zero_bits, rhi, rlo);
    else sqdd_e8_pair<FMT>(hi, lo, c.e8, rhi, rlo);
}

// exponent of RN(fmax / amax) for fmax = 1.75 * 2^k (448, 57344) or 1.875 * 2^2 (7.5)
// without the division: amax = m * 2^ea gives (c / m) * 2^(k - ea), and c / m < 1
// exactly when m > c (no float of either input type rounds c / m up to 1).  Valid for
// a normal, finite, non-zero amax; `bits` is its binary32 pattern.
template <int FMT>
__device__ __forceinline__ int e8_of_amax(uint32_t bits) {
    constexpr int k = (FMT == kE4M3) ? 8 : (FMT == kE5M2 ? 15 : (FMT == kE3M2 ? 4 : 2));
    constexpr uint32_t cman = (FMT == kE2M3) ? 0x700000u : 0x600000u;  // 1.875 / 1.75
    const int ea = (int)(bits >> 23) - 127;
    return k - ea - ((bits & 0x7FFFFFu) > cman ? 1 : 0);
}

// q / x for a float q of about the magnitude of x (or zero) and a bf16-valued x,
// 2^-64 <= |x| < 2^64 (so that the residual below stays a normal number): exactly RN(q / x).
// With r within one ulp of 1/x, q0 = q * r is within a few ulps of the quotient; x has
// 8 significant bits, so the residual q - x*q0 is exact in the fma, and q0 + rem * r
// differs from the true quotient by less than 2^-20 ulp, while a quotient by an 8-bit
// divisor is never closer than 2^-10 ulp to a rounding boundary: one correction step
// rounds correctly.
__device__ __forceinline__ float rcp_fast(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float div_by_bf16(float q, float x, float r) {
    const float q0 = __fmul_rn(q, r);
    const float rem = __fmaf_rn(-x, q0, q);
    return __fmaf_rn(rem, r, q0);
}
// The same quotient for a bf16-valued x of ANY magnitude (subnormal to 2^127) and a
// numerator of comparable or smaller magnitude: both are first multiplied by the power
// of two that brings x into [2^-6, 2], which changes neither operand's significand nor
// the quotient, and keeps every intermediate a normal number.
__device__ __forceinline__ float div_by_bf16_any(float num, float x) {
    int k = 127 - (int)((f2u(x) >> 23) & 0xFFu);
    k = max(k, -126);
    const float s = u2f((uint32_t)(k + 127) << 23);
    const float xs = __fmul_rn(x, s);
    return div_by_bf16(__fmul_rn(num, s), xs, rcp_fast(xs));
}
__device__ __forceinline__ bool bf16_div_safe(float x) { return (f2u(x) & 0x7FFFFFFFu) - 0x1F800000u < 0x40000000u; }

// packed bf16 magnitude helpers: both halves of a word at once
__device__ __forceinline__ uint32_t mag2(uint32_t w) { return w & 0x7FFF7FFFu; }
// number of non-zero halves of a magnitude word (each half <= 0x7FFF, so adding 0x7FFF
// sets bit 15 exactly when the half is non-zero and never carries across)
__device__ __forceinline__ int nnz2(uint32_t m) { return __popc((m + 0x7FFF7FFFu) & 0x80008000u); }
// packed 16-bit integer min / max: single instructions on this architecture
__device__ __forceinline__ uint32_t umax16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("max.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t umin16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("min.u16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t umax16x2_3(uint32_t a, uint32_t b, uint32_t c) { return __vimax3_u16x2(a, b, c); }
__device__ __forceinline__ uint32_t smin16x2_3(uint32_t a, uint32_t b, uint32_t c) { return __vimin3_s16x2(a, b, c); }
// bytes 1 and 3 of a and of b, each replaced by eight copies of its top bit
__device__ __forceinline__ uint32_t top_bits_to_bytes(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, 0xFDB9;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
// packed maximum of the four magnitude words of a 16-byte vector of bf16
__device__ __forceinline__ uint32_t umax16x2_vec(uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3) {
    return umax16x2(umax16x2_3(m0, m1, m2), m3);
}
__device__ __forceinline__ uint32_t hmax_halves(uint32_t m) { return max(m & 0xFFFFu, m >> 16); }

template <int FMT>
__device__ __forceinline__ float fmt_max() {
    if constexpr (FMT == kE4M3) return 448.0f;
    else if constexpr (FMT == kE5M2) return 57344.0f;
    else if constexpr (FMT == kE3M2) return 28.0f;
    else return 7.5f;
}

// ----------------------------------------------------------------------------
// element access: bf16 (two per 32-bit word) or binary32 (extension)
// ----------------------------------------------------------------------------
// A "word" is the pair of elements (2w, 2w+1); HI is element 2w+1.
struct Bf16 {
    using vec_t = uint4;                 // 16 bytes = 4 words = 8 elements
    static constexpr int kWordsPerVec = 4;
    static constexpr int kBytesPerElem = 2;
    __device__ static __forceinline__ void unpack(const vec_t& v, int k, float& hi, float& lo) {
        const uint32_t w = (k == 0) ? v.x : (k == 1) ? v.y : (k == 2) ? v.z : v.w;
        hi = bf16_hi(w);
        lo = bf16_lo(w);
    }
    __device__ static __forceinline__ void pack(vec_t& v, int k, float hi, float lo) {
        const uint32_t w = pack_bf16(hi, lo);
        if (k == 0) v.x = w; else if (k == 1) v.y = w; else if (k == 2) v.z = w; else v.w = w;
    }
};
struct Fp32 {
    using vec_t = float4;                // 16 bytes = 2 words = 4 elements
    static constexpr int kWordsPerVec = 2;
    static constexpr int kBytesPerElem = 4;
    __device__ static __forceinline__ void unpack(const vec_t& v, int k, float& hi, float& lo) {
        if (k == 0) { lo = v.x; hi = v.y; } else { lo = v.z; hi = v.w; }
    }
    __device__ static __forceinline__ void pack(vec_t& v, int k, float hi, float lo) {
        if (k == 0) { v.x = lo; v.y = hi; } else { v.z = lo; v.w = hi; }
    }
};

template <typename V>
__device__ __forceinline__ V ld_stream(const V* p) { return __ldcs(p); }   // read once: evict-first
template <typename V>
__device__ __forceinline__ V ld_keep(const V* p) { return __ldg(p); }      // will be read again
template <typename V>
__device__ __forceinline__ void st_stream(V* p, const V& v) { __stcs(p, v); }

// ----------------------------------------------------------------------------
// reductions
// ----------------------------------------------------------------------------
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// ref: 399-405.  The ORDER of these additions is part of the result: lane l adds
// the value of lane l+off for off = 16, 8, 4, 2, 1; only lane 0's sum is used.
__device__ __forceinline__ float warp_sum_ordered(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_down_sync(0xFFFFFFFFu, v, o));
    return v;
}

// Error sums over a virtual CTA of NL logical threads whose partial sums live VW to a
// physical lane: logical thread t = VW * p + k sits in slot k of physical lane p (p
// counted inside an aligned group of NL / VW lanes).  Reproduces, for logical lane 0
// of each logical warp (32 logical threads = 32 / VW physical lanes), the sum that
// warp_sum_ordered would give if every logical thread were a real lane.
template <int VW>
__device__ __forceinline__ float logical_warp_sum(float (&acc)[VW]) {
    static_assert(VW == 1 || VW == 2 || VW == 4, "words per lane");
#pragma unroll
    for (int o = 16; o >= VW; o >>= 1) {
#pragma unroll
        for (int k = 0; k < VW; ++k) acc[k] = __fadd_rn(acc[k], __shfl_down_sync(0xFFFFFFFFu, acc[k], o / VW));
    }
    if constexpr (VW == 4) {
        acc[0] = __fadd_rn(acc[0], acc[2]);
        acc[1] = __fadd_rn(acc[1], acc[3]);
    }
    if constexpr (VW >= 2) acc[0] = __fadd_rn(acc[0], acc[1]);
    return acc[0];
}

}  // namespace morb
