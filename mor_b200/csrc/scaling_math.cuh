// Per-element arithmetic of the tensor-scaled pipelines (fake_quantize_block_scaling and
// fake_quantize_channel_scaling; ref: 1059-1176, 1633-1752), shared by the kernels of
// fq_scaling.cu and fq_resident.cu.
#pragma once

#include "kernels.cuh"

namespace morb {
namespace {

// ref: 1059-1093.  All four strategies; the block amax is floored at 1e-35.
__device__ __forceinline__ float scaling_factor(int ss, float gamax, float bamax) {
    if (bamax < 1e-35f) bamax = 1e-35f;
    if (ss == 1) {
        const uint32_t gman = f2u(__fdiv_rn(448.0f, gamax)) & 0x007FFFFFu;
        const uint32_t bb = f2u(__fdiv_rn(448.0f, bamax));
        const float adj = u2f((bb & 0xFF800000u) | gman);
        return (gman <= (bb & 0x007FFFFFu)) ? adj : __fdiv_rn(adj, 2.0f);
    }
    if (ss == 2 || ss == 3) return __fdiv_rn(448.0f, bamax);
    if (ss == 4 && gamax > 0.0f) return __fdiv_rn(448.0f, gamax);
    return 1.0f;
}

__device__ __forceinline__ float read_gamax(const ScalarsWs* ws, const float* ext) {
    return ext ? *ext : u2f(ws->gamax_bits);
}
// may the four-instruction quotient by a bf16 value be used for the whole tensor?  (amax
// pass: no non-zero magnitude below 2^-90 and no NaN; here: nothing at or above 2^90)
template <typename T>
__device__ __forceinline__ bool fast_div_ok(const ScalarsWs* ws) {
    if constexpr (T::kBytesPerElem != 2) return false;
    else return ws->div_unsafe == 0u && ws->gamax_bits < 0x6C800000u;
}

// One element pair of block_e4m3_relative_error (ref: 1133-1162).  ss_mode 2 is the
// one that takes the power-of-two path: the reference tests `T_SCALING_STRATEGY ==
// SF_E8` and SF_E8 is the enumerator 2 of another enum.  Zeros are skipped by the
// reference: they are written back as +0 and add no error.
//
// Three ways to the same bits:
//   Lut   scale is a binary32 number shared by many elements: dequantised value =
//         table[code], the table filled once with the exact division q / scale;
//   Div   same scale kind, too few elements per scale to pay for a table;
//   E8    power-of-two scale: two multiplies (or the literal exponent-field form
//         outside the range where they are provably identical).
struct PathLut { const float* lut; float sf; };
// Scales that share their significand and differ by a power of two (the global-mantissa rule,
// ref: 1067-1076, gives every block the significand of 448 / global_amax): one table for the
// significand alone, `descale` = 2^-(exponent of sf).  RN(q / (m 2^e)) = RN(q / m) 2^-e as long as
// nothing leaves the normal range, which the caller checks from the exponent of sf.
struct PathLutExp { const float* lut; float sf; float descale; };
struct PathDiv { float sf; };
struct PathE8 { E8Consts c; };

__device__ __forceinline__ void dequant_pair(const PathLut& p, float hi, float lo, float& dh, float& dl) {
    const uint32_t c = cvt_codes<kE4M3>(__fmul_rn(hi, p.sf), __fmul_rn(lo, p.sf));
    dh = p.lut[c >> 8];
    dl = p.lut[c & 0xFFu];
}
__device__ __forceinline__ void dequant_pair(const PathLutExp& p, float hi, float lo, float& dh, float& dl) {
    const uint32_t c = cvt_codes<kE4M3>(__fmul_rn(hi, p.sf), __fmul_rn(lo, p.sf));
    dh = __fmul_rn(p.lut[c >> 8], p.descale);
    dl = __fmul_rn(p.lut[c & 0xFFu], p.descale);
}
__device__ __forceinline__ void dequant_pair(const PathDiv& p, float hi, float lo, float& dh, float& dl) {
    sqdd_fp32_pair<kE4M3>(hi, lo, p.sf, dh, dl);
    dh = canon_nan(dh);
    dl = canon_nan(dl);
}
__device__ __forceinline__ void dequant_pair(const PathE8& p, float hi, float lo, float& dh, float& dl) {
    sqdd_e8_pair_auto<kE4M3>(hi, lo, p.c, dh, dl);
}
template <typename P> struct PathTraits { static constexpr bool kExactBf16 = false; };
template <> struct PathTraits<PathE8> { static constexpr bool kExactBf16 = true; };

// table[code] = RN(dequant(code) / sf), NaNs canonicalised so that the add-and-shift
// bf16 rounding reproduces the reference's result for them
__device__ __forceinline__ void fill_lut32(float* lut, float sf, int tid, int nthreads) {
    for (int c = tid; c < 256; c += nthreads)
        lut[c] = canon_nan(__fdiv_rn(h_lo_to_f32(codes_to_h2<kE4M3>((uint32_t)c)), sf));
}

// |(d - x) / x| for x != 0 (ref: 1143, 1154).  Zero elements are skipped by the
// reference: no error, written back as +0; handled with selects, not branches.
// DIV selects how the exact quotient is formed:
//   kDivIeee     x is a binary32 value: the IEEE division;
//   kDivBf16     x carries a bf16 value and the amax pass found every non-zero magnitude
//                of the tensor inside [2^-90, 2^90): four instructions (div_by_bf16);
//   kDivBf16Any  x carries a bf16 value of any magnitude: operands pre-scaled by a power
//                of two, then the same four instructions.
enum { kDivIeee = 0, kDivBf16 = 1, kDivBf16Any = 2 };

template <int DIV, typename P, bool NOZERO = false>
__device__ __forceinline__ void err_pair(const P& path, float hi, float lo, float& dh, float& dl, float& eh,
                                         float& el) {
    dequant_pair(path, hi, lo, dh, dl);
    if constexpr (NOZERO) {  // the amax pass counted as many non-zero elements as the block has
        if constexpr (DIV == kDivBf16) {
            eh = fabsf(div_by_bf16(__fsub_rn(dh, hi), hi, rcp_fast(hi)));
            el = fabsf(div_by_bf16(__fsub_rn(dl, lo), lo, rcp_fast(lo)));
        } else if constexpr (DIV == kDivBf16Any) {
            eh = fabsf(div_by_bf16_any(__fsub_rn(dh, hi), hi));
            el = fabsf(div_by_bf16_any(__fsub_rn(dl, lo), lo));
        } else {
            eh = fabsf(__fdiv_rn(__fsub_rn(dh, hi), hi));
            el = fabsf(__fdiv_rn(__fsub_rn(dl, lo), lo));
        }
        return;
    }
    const bool zh = hi == 0.0f, zl = lo == 0.0f;
    if constexpr (DIV == kDivBf16) {
        eh = fabsf(div_by_bf16(__fsub_rn(dh, hi), hi, rcp_fast(hi)));
        el = fabsf(div_by_bf16(__fsub_rn(dl, lo), lo, rcp_fast(lo)));
    } else if constexpr (DIV == kDivBf16Any) {
        eh = fabsf(div_by_bf16_any(__fsub_rn(dh, hi), hi));
        el = fabsf(div_by_bf16_any(__fsub_rn(dl, lo), lo));
    } else {
        eh = fabsf(__fdiv_rn(__fsub_rn(dh, hi), zh ? 1.0f : hi));
        el = fabsf(__fdiv_rn(__fsub_rn(dl, lo), zl ? 1.0f : lo));
    }
    eh = zh ? 0.0f : eh;
    el = zl ? 0.0f : el;
    dh = zh ? 0.0f : dh;
    dl = zl ? 0.0f : dl;
}

// process one 16-byte vector: VW logical threads, errors added high half first
template <typename T, typename P, bool STORE, int DIV, bool NOZERO = false>
__device__ __forceinline__ void err_vec(const P& path, const typename T::vec_t& v, typename T::vec_t& o,
                                        float (&acc)[T::kWordsPerVec]) {
#pragma unroll
    for (int k = 0; k < T::kWordsPerVec; ++k) {
        float hi, lo, dh, dl, eh, el;
        T::unpack(v, k, hi, lo);
        err_pair<DIV, P, NOZERO>(path, hi, lo, dh, dl, eh, el);
        acc[k] = __fadd_rn(acc[k], eh);
        acc[k] = __fadd_rn(acc[k], el);
        if constexpr (STORE) {
            if constexpr (T::kBytesPerElem == 2) {
                uint32_t w;
                if constexpr (PathTraits<P>::kExactBf16) w = path.c.fast ? pack_bf16_trunc(dh, dl) : pack_bf16(dh, dl);
                else w = pack_bf16_round(dh, dl);
                if (k == 0) o.x = w; else if (k == 1) o.y = w; else if (k == 2) o.z = w; else o.w = w;
            } else {
                T::pack(o, k, dh, dl);
            }
        }
    }
}
// same, separate sums for the high and the low halves (channel kernels, ref: 1694-1748)
template <typename T, typename P, bool STORE, int DIV, bool NOZERO = false>
__device__ __forceinline__ void err_vec_split(const P& path, const typename T::vec_t& v, typename T::vec_t& o,
                                              float (&eh)[T::kWordsPerVec], float (&el)[T::kWordsPerVec]) {
#pragma unroll
    for (int k = 0; k < T::kWordsPerVec; ++k) {
        float hi, lo, dh, dl, e_h, e_l;
        T::unpack(v, k, hi, lo);
        err_pair<DIV, P, NOZERO>(path, hi, lo, dh, dl, e_h, e_l);
        eh[k] = __fadd_rn(eh[k], e_h);
        el[k] = __fadd_rn(el[k], e_l);
        if constexpr (STORE) {
            if constexpr (T::kBytesPerElem == 2) {
                uint32_t w;
                if constexpr (PathTraits<P>::kExactBf16) w = path.c.fast ? pack_bf16_trunc(dh, dl) : pack_bf16(dh, dl);
                else w = pack_bf16_round(dh, dl);
                if (k == 0) o.x = w; else if (k == 1) o.y = w; else if (k == 2) o.z = w; else o.w = w;
            } else {
                T::pack(o, k, dh, dl);
            }
        }
    }
}

// the pair of elements (2w, 2w + 1) as one word: 4 bytes of bf16, 8 bytes of binary32
template <typename T> struct PairWord;
template <> struct PairWord<Bf16> {
    using type = uint32_t;
    __device__ static __forceinline__ void unpack(uint32_t w, float& hi, float& lo) { hi = bf16_hi(w); lo = bf16_lo(w); }
    template <typename P>
    __device__ static __forceinline__ uint32_t pack(const P& path, float dh, float dl) {
        if constexpr (PathTraits<P>::kExactBf16) return path.c.fast ? pack_bf16_trunc(dh, dl) : pack_bf16(dh, dl);
        else return pack_bf16_round(dh, dl);
    }
};
template <> struct PairWord<Fp32> {
    using type = float2;
    __device__ static __forceinline__ void unpack(float2 w, float& hi, float& lo) { hi = w.y; lo = w.x; }
    template <typename P>
    __device__ static __forceinline__ float2 pack(const P&, float dh, float dl) { return make_float2(dl, dh); }
};

}  // namespace
}  // namespace morb
