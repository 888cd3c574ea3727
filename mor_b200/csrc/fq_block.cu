// fake_quantize with a scale per (brows x bcols) block: MoR's per-block choice of
// representation and the fixed E4M3 / E5M2 block modes (ref: 407-852).
//
//   fq_tile128_kernel  128 x 128 bf16 blocks: the 32 KiB tile is read from HBM once,
//                      by TMA into shared memory, and stays there through the
//                      amax/amin pass, the optional two-format error pass and the
//                      cast; one HBM read + one HBM write per element.
//   fq_block_generic_kernel  any block shape, ragged edges, bf16 or binary32; rereads
//                      the block (L1/L2 hits) instead of caching it.
//
// The error pass compares two float sums, so both kernels add in the order of the
// reference's CTA of 16 x 32 threads (one thread per 32-bit word, rows outer, words
// inner, (e_high + e_low) per word, shfl_down trees); see logical_warp_sum().
#include <cuda.h>

#include <type_traits>

#include "kernels.cuh"
#include "tma.cuh"

namespace morb {

namespace {

enum { QM_MOR = 1, QM_BLOCK_E4M3 = 2, QM_BLOCK_E5M2 = 3 };
enum { Q_E4M3 = 1, Q_E5M2 = 2, Q_BF16 = 3, Q_E2M3 = 4, Q_E4M3_SMALL = 11, Q_E5M2_SMALL = 12 };
enum { NEED_ERRORS = -1 };

// ref: 610-682 up to the point where the error sums are needed.
__device__ __forceinline__ int choose_by_range(float amax, float amin, float clamp, bool dynamic_range_mode) {
    float range = 0.0f;
    if (amax == 0.0f) { amax = clamp; range = 1.0f; }
    if (range == 0.0f) range = __fdiv_rn(amax, amin);
    const float e4_range = dynamic_range_mode ? 28672.0f : 114688.0f;
    if (range <= 7.5f) return Q_E2M3;
    if (range <= e4_range) return amax <= clamp ? Q_E4M3_SMALL : Q_E4M3;
    if (range <= 939524096.0f) {
        if (dynamic_range_mode) return amax <= clamp ? Q_E5M2_SMALL : Q_E5M2;
        return NEED_ERRORS;
    }
    return Q_BF16;
}
__device__ __forceinline__ int choose_by_error(float err4, float err5, float amax, float clamp) {
    if (err4 <= err5) return amax <= clamp ? Q_E4M3_SMALL : Q_E4M3;
    return Q_BF16;  // the error criterion never selects E5M2 (ref: 672-674)
}
__device__ __forceinline__ int repr_to_fmt(int repr) {
    if (repr == Q_E2M3) return kE2M3;
    if (repr == Q_E4M3 || repr == Q_E4M3_SMALL) return kE4M3;
    if (repr == Q_E5M2 || repr == Q_E5M2_SMALL) return kE5M2;
    return -1;
}

// ref: 504-541: e = |q/x - 1| for x != 0, (e_high + e_low) per word, both formats.
template <int SF>
__device__ __forceinline__ void word_errors(float hi, float lo, float s4, float s5, float& e4, float& e5) {
    float qh, ql, eh, el;
    sqdd_pair<kE4M3, SF>(hi, lo, s4, qh, ql);
    eh = (hi != 0.0f) ? fabsf(__fsub_rn(__fdiv_rn(qh, hi), 1.0f)) : 0.0f;
    el = (lo != 0.0f) ? fabsf(__fsub_rn(__fdiv_rn(ql, lo), 1.0f)) : 0.0f;
    e4 = __fadd_rn(eh, el);
    sqdd_pair<kE5M2, SF>(hi, lo, s5, qh, ql);
    eh = (hi != 0.0f) ? fabsf(__fsub_rn(__fdiv_rn(qh, hi), 1.0f)) : 0.0f;
    el = (lo != 0.0f) ? fabsf(__fsub_rn(__fdiv_rn(ql, lo), 1.0f)) : 0.0f;
    e5 = __fadd_rn(eh, el);
}

template <int SF>
__device__ __forceinline__ void cast_pair(int fmt, float hi, float lo, float s, float& rh, float& rl) {
    if (fmt == kE4M3) sqdd_pair<kE4M3, SF>(hi, lo, s, rh, rl);
    else if (fmt == kE5M2) sqdd_pair<kE5M2, SF>(hi, lo, s, rh, rl);
    else sqdd_pair<kE2M3, SF>(hi, lo, s, rh, rl);
}

// ---------------------------------------------------------------------------------
// 128 x 128 bf16 tile staged in shared memory by TMA
// ---------------------------------------------------------------------------------
// One CTA of 128 threads per tile.  Thread 0 issues four cp.async.bulk.tensor.2d loads
// (column strips of 32 elements = 64 bytes x 128 rows) that land as strip-major
// [4][128][64 B] in shared memory and signal an mbarrier; several CTAs per SM overlap
// one tile's load with another's arithmetic.  Lane (a, ty) owns the reference's
// logical threads tx = 4a..4a+3 of row ty: its 16-byte chunk of strip i, row ty + 32 j
// holds words tx + 16 i, and a warp's eight rows x four chunks are 512 contiguous
// bytes, so every shared-memory access is conflict-free.  The passes (amax/amin, the
// optional two-format error sums, the cast) walk the tile with rolled loops; results
// go from registers straight to global memory with 16-byte stores.

constexpr int kTileBytes = 128 * 128 * 2;
template <int SF>
struct ErrCtx {
    const float* lut4;  // SF_FP32: RN(dequant(code) / s) tables
    const float* lut5;
    float s4, s5;
    E8Consts c4, c5;    // SF_E8
};

// |q4/x - 1| and |q5/x - 1| for one element (ref: 504-541); zero elements add nothing
template <int SF, bool SAFE>
__device__ __forceinline__ void word_errors_fast(const ErrCtx<SF>& e, float hi, float lo, float& e4, float& e5) {
    float q4h, q4l, q5h, q5l;
    if constexpr (SF == kSfFp32) {
        const uint32_t c4 = cvt_codes<kE4M3>(__fmul_rn(hi, e.s4), __fmul_rn(lo, e.s4));
        const uint32_t c5 = cvt_codes<kE5M2>(__fmul_rn(hi, e.s5), __fmul_rn(lo, e.s5));
        q4h = e.lut4[c4 >> 8]; q4l = e.lut4[c4 & 0xFFu];
        q5h = e.lut5[c5 >> 8]; q5l = e.lut5[c5 & 0xFFu];
    } else {
        sqdd_e8_pair_auto<kE4M3>(hi, lo, e.c4, q4h, q4l);
        sqdd_e8_pair_auto<kE5M2>(hi, lo, e.c5, q5h, q5l);
    }
    float e4h = 0.0f, e4l = 0.0f, e5h = 0.0f, e5l = 0.0f;
    if constexpr (SAFE) {
        // branch-free: a zero element yields NaN garbage that the selects discard
        const float rh = rcp_fast(hi), rl = rcp_fast(lo);
        const bool zh = hi == 0.0f, zl = lo == 0.0f;
        e4h = fabsf(__fsub_rn(div_by_bf16(q4h, hi, rh), 1.0f));
        e5h = fabsf(__fsub_rn(div_by_bf16(q5h, hi, rh), 1.0f));
        e4l = fabsf(__fsub_rn(div_by_bf16(q4l, lo, rl), 1.0f));
        e5l = fabsf(__fsub_rn(div_by_bf16(q5l, lo, rl), 1.0f));
        e4h = zh ? 0.0f : e4h; e5h = zh ? 0.0f : e5h;
        e4l = zl ? 0.0f : e4l; e5l = zl ? 0.0f : e5l;
    } else {
        // magnitudes outside the short form's range: same quotient after a power-of-two pre-scale
        const bool zh = hi == 0.0f, zl = lo == 0.0f;
        e4h = fabsf(__fsub_rn(div_by_bf16_any(q4h, hi), 1.0f));
        e5h = fabsf(__fsub_rn(div_by_bf16_any(q5h, hi), 1.0f));
        e4l = fabsf(__fsub_rn(div_by_bf16_any(q4l, lo), 1.0f));
        e5l = fabsf(__fsub_rn(div_by_bf16_any(q5l, lo), 1.0f));
        e4h = zh ? 0.0f : e4h; e5h = zh ? 0.0f : e5h;
        e4l = zl ? 0.0f : e4l; e5l = zl ? 0.0f : e5l;
    }
    e4 = __fadd_rn(e4h, e4l);
    e5 = __fadd_rn(e5h, e5l);
}

template <int FMT>
__device__ __forceinline__ void fill_lut16(uint16_t* lut, float s, int tid) {
    constexpr int NCODES = (FMT == kE2M3) ? 64 : 256;
    for (int c = tid; c < NCODES; c += 128) {
        float q = h_lo_to_f32(codes_to_h2<FMT>((uint32_t)c));
        if (FMT == kE2M3 && q == 0.0f) q = 0.0f;  // the custom cast returns +0
        lut[c] = (uint16_t)f32_to_bf16_bits(__fdiv_rn(q, s));
    }
}
template <int FMT>
__device__ __forceinline__ void fill_lut32t(float* lut, float s, int tid) {
    for (int c = tid; c < 256; c += 128) lut[c] = __fdiv_rn(h_lo_to_f32(codes_to_h2<FMT>((uint32_t)c)), s);
}
template <int FMT>
__device__ __forceinline__ uint32_t lut_word(const uint16_t* lut, uint32_t w, float s) {
    const uint32_t c = cvt_codes<FMT>(__fmul_rn(bf16_hi(w), s), __fmul_rn(bf16_lo(w), s));
    return __byte_perm((uint32_t)lut[c & 0xFFu], (uint32_t)lut[c >> 8], 0x5410);
}
template <int FMT>
__device__ __forceinline__ uint32_t e8_word(uint32_t w, const E8Consts& c) {
    float rh, rl;
    sqdd_e8_pair_auto<FMT>(bf16_hi(w), bf16_lo(w), c, rh, rl);
    return c.fast ? pack_bf16_trunc(rh, rl) : pack_bf16(rh, rl);
}

template <int SF>
__global__ void __launch_bounds__(128)
fq_tile128_kernel(const __grid_constant__ CUtensorMap tmap, uint4* __restrict__ out, int32_t* __restrict__ meta,
                  int64_t cols_vec, int blocks_x, float clamp, int qmode, int dyn_mode) {
    extern __shared__ __align__(128) uint8_t s_tile[];  // [4 strips][128 rows][64 B]
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ float s_red[2][4];
    __shared__ float s_w4[16], s_w5[16];
    __shared__ float s_tot[2];
    __shared__ __align__(16) float s_lut4[256];
    __shared__ __align__(16) float s_lut5[256];
    uint16_t* s_lut16 = reinterpret_cast<uint16_t*>(s_lut4);  // the cast table reuses the error tables' space
    const int tid = threadIdx.x, a = tid & 3, ty = tid >> 2, lane = tid & 31, wid = tid >> 5;
    const int64_t b = blockIdx.x;
    const int bx = (int)(b % blocks_x), by = (int)(b / blocks_x);

    if (tid == 0) mbar_init(&s_bar, 1);
    __syncthreads();
    if (tid == 0) {
        mbar_expect_tx(&s_bar, kTileBytes);
#pragma unroll
        for (int sidx = 0; sidx < 4; ++sidx) tma_load_2d(s_tile + sidx * 8192, &tmap, bx * 128 + sidx * 32, by * 128, &s_bar);
    }
    if (!mbar_wait_bounded(&s_bar, 0)) {
        // the load did not complete: report it in meta, give the copy one more bounded
        // chance to land before this CTA's shared memory is handed to the next one
        if (tid == 0) meta[b] = -1;
        mbar_wait_bounded(&s_bar, 0);
        return;
    }
    const uint4* tile = reinterpret_cast<const uint4*>(s_tile);
    auto chunk = [&](int j, int i) -> uint4 { return tile[i * 512 + (ty + 32 * j) * 4 + a]; };

    // amax and smallest non-zero magnitude (ref: 407-485); bf16 magnitudes order like
    // their 15-bit patterns, and "pattern - 1" as unsigned sends zero to the top.
    uint32_t mx = 0u, mn = 0x7F7Eu;  // 0x7F7F - 1: the reference starts amin at the bf16 maximum
    auto scan = [&](uint32_t w) {
        const uint32_t lo = w & 0x7FFFu, hi = (w >> 16) & 0x7FFFu;
        // NaN patterns are ignored by the reference's fmaxf/fminf
        const uint32_t lo_v = lo > 0x7F80u ? 0u : lo, hi_v = hi > 0x7F80u ? 0u : hi;
        mx = max(mx, max(lo_v, hi_v));
        mn = min(mn, min(lo_v - 1u, hi_v - 1u));
    };
#pragma unroll 4
    for (int n = 0; n < 16; ++n) {
        const uint4 v = chunk(n >> 2, n & 3);
        scan(v.x); scan(v.y); scan(v.z); scan(v.w);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        mn = min(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, o));
    }
    if (lane == 0) { s_red[0][wid] = u2f(mx << 16); s_red[1][wid] = u2f((mn + 1u) << 16); }
    __syncthreads();
    const float amax = fmaxf(fmaxf(s_red[0][0], s_red[0][1]), fmaxf(s_red[0][2], s_red[0][3]));
    const float amin = fminf(fminf(s_red[1][0], s_red[1][1]), fminf(s_red[1][2], s_red[1][3]));

    int repr = 0, code = 3, fmt = -1;
    if (qmode == QM_MOR) {
        repr = choose_by_range(amax, amin, clamp, dyn_mode != 0);
        if (repr == NEED_ERRORS) {
            ErrCtx<SF> e;
            e.s4 = __fdiv_rn(448.0f, amax);
            e.s5 = __fdiv_rn(57344.0f, amax);
            e.lut4 = s_lut4; e.lut5 = s_lut5;
            if constexpr (SF == kSfFp32) {
                fill_lut32t<kE4M3>(s_lut4, e.s4, tid);
                fill_lut32t<kE5M2>(s_lut5, e.s5, tid);
                __syncthreads();
            } else {
                e.c4 = e8_consts(e.s4);
                e.c5 = e8_consts(e.s5);
            }
            // every non-zero magnitude of the block lies in [amin, amax]
            const bool safe = bf16_div_safe(amin) && bf16_div_safe(amax);
            float a4[4] = {0.f, 0.f, 0.f, 0.f}, a5[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
            for (int n = 0; n < 16; ++n) {  // rows outer (j = n / 4), words inner (i = n % 4)
                const uint4 v = chunk(n >> 2, n & 3);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float e4, e5;
                    if (safe) word_errors_fast<SF, true>(e, bf16_hi(w[k]), bf16_lo(w[k]), e4, e5);
                    else word_errors_fast<SF, false>(e, bf16_hi(w[k]), bf16_lo(w[k]), e4, e5);
                    a4[k] = __fadd_rn(a4[k], e4);
                    a5[k] = __fadd_rn(a5[k], e5);
                }
            }
            const float w4 = logical_warp_sum<4>(a4), w5 = logical_warp_sum<4>(a5);
            if ((tid & 7) == 0) { s_w4[tid >> 3] = w4; s_w5[tid >> 3] = w5; }
            __syncthreads();
            if (wid == 0) {
                const float t4 = warp_sum_ordered(lane < 16 ? s_w4[lane] : 0.0f);
                const float t5 = warp_sum_ordered(lane < 16 ? s_w5[lane] : 0.0f);
                if (lane == 0) { s_tot[0] = t4; s_tot[1] = t5; }
            }
            __syncthreads();
            repr = choose_by_error(s_tot[0], s_tot[1], amax, clamp);
        }
        code = repr;
        fmt = repr_to_fmt(repr);
    } else if (qmode == QM_BLOCK_E4M3) { code = 1; fmt = kE4M3; }
    else if (qmode == QM_BLOCK_E5M2) { code = 2; fmt = kE5M2; }
    if (tid == 0) meta[b] = code;
    if (!(amax > 0.0f)) fmt = -1;  // all-zero block: copied through (ref: 759, 773, 787, 802, 814)

    uint4* dst = out + ((int64_t)by * 128) * cols_vec + (int64_t)bx * 16;
    auto store = [&](int n, const uint4& v) { st_stream(dst + (int64_t)(ty + 32 * (n >> 2)) * cols_vec + 4 * (n & 3) + a, v); };
    if (fmt < 0) {
#pragma unroll 4
        for (int n = 0; n < 16; ++n) store(n, chunk(n >> 2, n & 3));
        return;
    }
    const float s = __fdiv_rn(fmt == kE2M3 ? 7.5f : (fmt == kE4M3 ? 448.0f : 57344.0f), amax);
    if constexpr (SF == kSfFp32) {
        if (fmt == kE4M3) fill_lut16<kE4M3>(s_lut16, s, tid);
        else if (fmt == kE5M2) fill_lut16<kE5M2>(s_lut16, s, tid);
        else fill_lut16<kE2M3>(s_lut16, s, tid);
        __syncthreads();
        auto cast_all = [&](auto fmt_tag) {
            constexpr int F = decltype(fmt_tag)::value;
#pragma unroll 2
            for (int n = 0; n < 16; ++n) {
                uint4 v = chunk(n >> 2, n & 3);
                v.x = lut_word<F>(s_lut16, v.x, s); v.y = lut_word<F>(s_lut16, v.y, s);
                v.z = lut_word<F>(s_lut16, v.z, s); v.w = lut_word<F>(s_lut16, v.w, s);
                store(n, v);
            }
        };
        if (fmt == kE4M3) cast_all(std::integral_constant<int, kE4M3>{});
        else if (fmt == kE5M2) cast_all(std::integral_constant<int, kE5M2>{});
        else cast_all(std::integral_constant<int, kE2M3>{});
    } else {
        const E8Consts c = e8_consts(s);
        auto cast_all = [&](auto fmt_tag) {
            constexpr int F = decltype(fmt_tag)::value;
#pragma unroll 2
            for (int n = 0; n < 16; ++n) {
                uint4 v = chunk(n >> 2, n & 3);
                v.x = e8_word<F>(v.x, c); v.y = e8_word<F>(v.y, c); v.z = e8_word<F>(v.z, c); v.w = e8_word<F>(v.w, c);
                store(n, v);
            }
        };
        if (fmt == kE4M3) cast_all(std::integral_constant<int, kE4M3>{});
        else if (fmt == kE5M2) cast_all(std::integral_constant<int, kE5M2>{});
        else cast_all(std::integral_constant<int, kE2M3>{});
    }
}

// ---------------------------------------------------------------------------------
// generic blocks
// ---------------------------------------------------------------------------------
template <typename T> struct WordOf;
template <> struct WordOf<Bf16> {
    using type = uint32_t;
    __device__ static __forceinline__ void unpack(uint32_t w, float& hi, float& lo) { hi = bf16_hi(w); lo = bf16_lo(w); }
    __device__ static __forceinline__ uint32_t pack(float hi, float lo) { return pack_bf16(hi, lo); }
};
template <> struct WordOf<Fp32> {
    using type = float2;
    __device__ static __forceinline__ void unpack(float2 w, float& hi, float& lo) { hi = w.y; lo = w.x; }
    __device__ static __forceinline__ float2 pack(float hi, float lo) { return make_float2(lo, hi); }
};

template <typename T, int SF>
__global__ void __launch_bounds__(256)
fq_block_generic_kernel(const typename WordOf<T>::type* __restrict__ in, typename WordOf<T>::type* __restrict__ out,
                        int32_t* __restrict__ meta, int64_t rows, int64_t colsw, int brows, int bcolsw,
                        int64_t blocks_x, float clamp, int qmode, int dyn_mode, int ltx, int lty) {
    using W = WordOf<T>;
    __shared__ float s_part4[1024], s_part5[1024];
    __shared__ float s_w4[32], s_w5[32];
    __shared__ float s_red[2][8];
    __shared__ float s_tot[2];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int64_t b = blockIdx.x;
    const int64_t r0 = (b / blocks_x) * brows, w0 = (b % blocks_x) * bcolsw;
    const int nr = (int)((r0 + brows <= rows ? r0 + brows : rows) - r0);
    const int nw = (int)((w0 + bcolsw <= colsw ? w0 + bcolsw : colsw) - w0);
    const int nwords = nr * nw;

    float amax = 0.0f, amin = u2f(0x7F7F0000u);
    for (int idx = tid; idx < nwords; idx += 256) {
        float hi, lo;
        W::unpack(in[(r0 + idx / nw) * colsw + w0 + idx % nw], hi, lo);
        const float ah = fabsf(hi), al = fabsf(lo);
        amax = fmaxf(amax, fmaxf(ah, al));
        if (ah > 0.0f) amin = fminf(amin, ah);
        if (al > 0.0f) amin = fminf(amin, al);
    }
    amax = warp_max(amax);
    amin = warp_min(amin);
    if (lane == 0) { s_red[0][wid] = amax; s_red[1][wid] = amin; }
    __syncthreads();
#pragma unroll
    for (int w = 0; w < 8; ++w) { amax = fmaxf(amax, s_red[0][w]); amin = fminf(amin, s_red[1][w]); }

    int repr = 0, code = 3, fmt = -1;
    if (qmode == QM_MOR) {
        repr = choose_by_range(amax, amin, clamp, dyn_mode != 0);
        if (repr == NEED_ERRORS) {
            const float s4 = __fdiv_rn(448.0f, amax), s5 = __fdiv_rn(57344.0f, amax);
            const int nl = ltx * lty;  // logical threads of the reference CTA (multiple of 32, <= 1024)
            for (int l = tid; l < nl; l += 256) {
                const int i = l % ltx, j = l / ltx;
                float a4 = 0.0f, a5 = 0.0f;
                for (int r = j; r < nr; r += lty)
                    for (int w = i; w < nw; w += ltx) {
                        float hi, lo, e4, e5;
                        W::unpack(in[(r0 + r) * colsw + w0 + w], hi, lo);
                        word_errors<SF>(hi, lo, s4, s5, e4, e5);
                        a4 = __fadd_rn(a4, e4);
                        a5 = __fadd_rn(a5, e5);
                    }
                s_part4[l] = a4;
                s_part5[l] = a5;
            }
            __syncthreads();
            const int nlw = nl / 32;
            for (int lw = wid; lw < nlw; lw += 8) {
                const float t4 = warp_sum_ordered(s_part4[lw * 32 + lane]);
                const float t5 = warp_sum_ordered(s_part5[lw * 32 + lane]);
                if (lane == 0) { s_w4[lw] = t4; s_w5[lw] = t5; }
            }
            __syncthreads();
            if (wid == 0) {
                const float t4 = warp_sum_ordered(lane < nlw ? s_w4[lane] : 0.0f);
                const float t5 = warp_sum_ordered(lane < nlw ? s_w5[lane] : 0.0f);
                if (lane == 0) { s_tot[0] = t4; s_tot[1] = t5; }
            }
            __syncthreads();
            repr = choose_by_error(s_tot[0], s_tot[1], amax, clamp);
        }
        code = repr;
        fmt = repr_to_fmt(repr);
    } else if (qmode == QM_BLOCK_E4M3) { code = 1; fmt = kE4M3; }
    else if (qmode == QM_BLOCK_E5M2) { code = 2; fmt = kE5M2; }
    if (tid == 0) meta[b] = code;
    if (!(amax > 0.0f)) fmt = -1;
    if (fmt < 0 && in == out) return;
    const float s = fmt >= 0 ? __fdiv_rn(fmt == kE2M3 ? 7.5f : (fmt == kE4M3 ? 448.0f : 57344.0f), amax) : 1.0f;
    for (int idx = tid; idx < nwords; idx += 256) {
        const int64_t off = (r0 + idx / nw) * colsw + w0 + idx % nw;
        typename W::type w = in[off];
        if (fmt >= 0) {
            float hi, lo, rh, rl;
            W::unpack(w, hi, lo);
            cast_pair<SF>(fmt, hi, lo, s, rh, rl);
            w = W::pack(rh, rl);
        }
        out[off] = w;
    }
}

}  // namespace

int launch_fq_block(const void* in, void* out, int is_fp32, int32_t* meta, int64_t rows, int64_t cols, int brows,
                    int bcols, float clamp, int quant_mode, int dynamic_range_mode, int sf_type, cudaStream_t st) {
    const int64_t colsw = cols / 2;
    const int bcolsw = bcols / 2;
    const int64_t bx = (colsw - 1) / bcolsw + 1, by = (rows - 1) / brows + 1, nb = bx * by;
    if (nb > 0x7FFFFFFF) return kErrTooLarge;
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    static const bool force_generic = getenv("MOR_B200_FORCE_GENERIC") != nullptr;
    if (!is_fp32 && brows == 128 && bcols == 128 && rows % 128 == 0 && cols % 128 == 0 && aligned && !force_generic &&
        rows < (int64_t(1) << 31) && cols < (int64_t(1) << 31)) {
        CUtensorMap map;
        if (make_tile_map(&map, in, rows, cols, 2, 32, 128)) {
            auto* o4 = static_cast<uint4*>(out);
            if (sf_type == kSfE8) fq_tile128_kernel<kSfE8><<<(unsigned)nb, 128, kTileBytes, st>>>(map, o4, meta, cols / 8, (int)bx, clamp, quant_mode, dynamic_range_mode);
            else fq_tile128_kernel<kSfFp32><<<(unsigned)nb, 128, kTileBytes, st>>>(map, o4, meta, cols / 8, (int)bx, clamp, quant_mode, dynamic_range_mode);
            return check_launch();
        }
    }
    // logical CTA of the reference (ref: 1770-1790), needed for the order of the error sums
    int ltx = 16, lty = 32;
    if ((int64_t)brows * bcols <= 1024) { ltx = bcolsw; lty = brows; }
    if (quant_mode == QM_MOR && (((ltx * lty) % 32) != 0 || ltx * lty > 1024)) return kErrUnsupportedShape;
#define MORB_GO(T, S) fq_block_generic_kernel<T, S><<<(unsigned)nb, 256, 0, st>>>(static_cast<const WordOf<T>::type*>(in), static_cast<WordOf<T>::type*>(out), meta, rows, colsw, brows, bcolsw, bx, clamp, quant_mode, dynamic_range_mode, ltx, lty)
    if (is_fp32) { if (sf_type == kSfE8) MORB_GO(Fp32, kSfE8); else MORB_GO(Fp32, kSfFp32); }
    else { if (sf_type == kSfE8) MORB_GO(Bf16, kSfE8); else MORB_GO(Bf16, kSfFp32); }
#undef MORB_GO
    return check_launch();
}

}  // namespace morb
