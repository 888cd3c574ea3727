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
template <int FMT>
__device__ __forceinline__ void quant_dequant_pair(float hi, float lo, float& qhi, float& qlo) {
    const uint32_t h2 = codes_to_h2<FMT>(cvt_codes<FMT>(hi, lo));
    qhi = h_hi_to_f32(h2);
    qlo = h_lo_to_f32(h2);
    if constexpr (FMT == kE2M3 || FMT == kE3M2) {
        if (qhi == 0.0f) qhi = 0.0f;  // -0 -> +0
        if (qlo == 0.0f) qlo = 0.0f;
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
