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
constexpr int kErrTableEntries = 2560;  // 20 rows of 128 magnitude patterns: 30 binades less the 11 folded ones, and slack
template <int SF>
struct ErrCtx {
    const float* lut4;  // SF_FP32: RN(dequant(code) / s) tables
    const float* lut5;
    float s4, s5;
    E8Consts c4, c5;    // SF_E8
};

// |q4/x - 1| and |q5/x - 1| for one element (ref: 504-541); zero elements add nothing
template <int SF, bool SAFE>
__device__ __forceinline__ void pair_errors(const ErrCtx<SF>& e, float hi, float lo, float& e4h, float& e4l,
                                            float& e5h, float& e5l) {
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
}
template <int SF, bool SAFE>
__device__ __forceinline__ void word_errors_fast(const ErrCtx<SF>& e, float hi, float lo, float& e4, float& e5) {
    float e4h, e4l, e5h, e5l;
    pair_errors<SF, SAFE>(e, hi, lo, e4h, e4l, e5h, e5l);
    e4 = __fadd_rn(e4h, e4l);
    e5 = __fadd_rn(e5h, e5l);
}

// (a.x + b.x, a.y + b.y), each sum rounded to nearest even as a single addition would be
__device__ __forceinline__ float2 add_f32x2(float2 a, float2 b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(*reinterpret_cast<const unsigned long long*>(&a)),
                                                "l"(*reinterpret_cast<const unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&r);
}
template <int FMT>
__device__ __forceinline__ void fill_lut16(uint16_t* lut, float s, int tid, int nthreads) {
    constexpr int NCODES = (FMT == kE2M3) ? 64 : 256;
    for (int c = tid; c < NCODES; c += nthreads) {
        float q = h_lo_to_f32(codes_to_h2<FMT>((uint32_t)c));
        if (FMT == kE2M3 && q == 0.0f) q = 0.0f;  // the custom cast returns +0
        lut[c] = (uint16_t)f32_to_bf16_bits(__fdiv_rn(q, s));
    }
}
template <int FMT>
__device__ __forceinline__ void fill_lut32t(float* lut, float s, int tid, int nthreads) {
    for (int c = tid; c < 256; c += nthreads) lut[c] = __fdiv_rn(h_lo_to_f32(codes_to_h2<FMT>((uint32_t)c)), s);
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

// VW = words of a strip row per thread: 4 (16-byte accesses, 128 threads) or 2 (8-byte accesses,
// 256 threads: the variant for the relative-error criterion, whose error table halves the number
// of CTAs an SM can hold).  Either way a thread owns VW logical threads of the reference's CTA.
template <int VW> struct TileVec;
template <> struct TileVec<4> { using type = uint4; };
template <> struct TileVec<2> { using type = uint2; };
template <int VW> __device__ __forceinline__ void tile_unpack(const typename TileVec<VW>::type& v, uint32_t (&w)[VW]);
template <> __device__ __forceinline__ void tile_unpack<4>(const uint4& v, uint32_t (&w)[4]) { w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
template <> __device__ __forceinline__ void tile_unpack<2>(const uint2& v, uint32_t (&w)[2]) { w[0] = v.x; w[1] = v.y; }
template <int VW> __device__ __forceinline__ typename TileVec<VW>::type tile_pack(const uint32_t (&w)[VW]);
template <> __device__ __forceinline__ uint4 tile_pack<4>(const uint32_t (&w)[4]) { return make_uint4(w[0], w[1], w[2], w[3]); }
template <> __device__ __forceinline__ uint2 tile_pack<2>(const uint32_t (&w)[2]) { return make_uint2(w[0], w[1]); }

template <int SF, int VW>
__global__ void __launch_bounds__(512 / VW, VW == 2 ? 4 : 7)
fq_tile128_kernel(const __grid_constant__ CUtensorMap tmap, typename TileVec<VW>::type* __restrict__ out, int32_t* __restrict__ meta,
                  int64_t cols_vec, int blocks_x, float clamp, int qmode, int dyn_mode, int table_entries) {
    extern __shared__ __align__(128) uint8_t s_tile[];  // [4 strips][128 rows][64 B], then the error table
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ float s_w4[16], s_w5[16];
    __shared__ float s_tot[2];
    __shared__ __align__(16) float s_lut4[256];
    __shared__ __align__(16) float s_lut5[256];
    uint16_t* s_lut16 = reinterpret_cast<uint16_t*>(s_lut4);  // the cast table reuses the error tables' space
    using V = typename TileVec<VW>::type;
    constexpr int LPR = 16 / VW;        // lanes per 64-byte strip row
    constexpr int NT = 32 * LPR;        // threads: 32 rows x LPR lanes per step
    constexpr int NW = NT / 32;
    const int tid = threadIdx.x, a = tid % LPR, ty = tid / LPR, lane = tid & 31, wid = tid >> 5;
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
    const V* tile = reinterpret_cast<const V*>(s_tile);
    auto chunk = [&](int j, int i) -> V { return tile[i * (128 * LPR) + (ty + 32 * j) * LPR + a]; };

    // amax and smallest non-zero magnitude (ref: 407-485) on packed words: one unsigned
    // 16-bit maximum of the magnitudes, and one signed 16-bit minimum of magnitude + 0x7FFF
    // (a zero becomes 0x7FFF, the largest; a magnitude m becomes 0x8000 + m - 1, ordered by
    // m).  NaN patterns, which the reference's fmaxf/fminf ignore, sort above infinity: a
    // tile that holds one is scanned again with the per-element form.
    //
    // RT (the 256-thread variant): the thread's 64 elements are read from shared memory once and stay in
    // registers for the passes that follow; the error pass then reuses the first half of the tile's space.
    constexpr bool RT = VW == 2;
    uint32_t tw[RT ? 16 : 1][VW];
    uint32_t pmx = 0u, pmn = 0x7FFF7FFFu;
    if constexpr (RT) {
#pragma unroll
        for (int n = 0; n < 16; ++n) tile_unpack<VW>(chunk(n >> 2, n & 3), tw[n]);
#pragma unroll
        for (int n = 0; n < 16; ++n) {
            const uint32_t m0 = mag2(tw[n][0]), m1 = mag2(tw[n][1]);
            pmx = umax16x2_3(pmx, m0, m1);
            pmn = smin16x2_3(pmn, m0 + 0x7FFF7FFFu, m1 + 0x7FFF7FFFu);
        }
    } else {
#pragma unroll 4
        for (int n = 0; n < 16; ++n) {
            uint32_t w[VW];
            tile_unpack<VW>(chunk(n >> 2, n & 3), w);
#pragma unroll
            for (int q = 0; q < VW; q += 2) {
                const uint32_t m0 = mag2(w[q]), m1 = mag2(w[q + 1]);
                pmx = umax16x2_3(pmx, m0, m1);
                pmn = smin16x2_3(pmn, m0 + 0x7FFF7FFFu, m1 + 0x7FFF7FFFu);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        pmx = umax16x2(pmx, __shfl_xor_sync(0xFFFFFFFFu, pmx, o));
        pmn = smin16x2_3(pmn, pmn, __shfl_xor_sync(0xFFFFFFFFu, pmn, o));
    }
    __shared__ uint32_t s_pk[2][NW];
    if (lane == 0) { s_pk[0][wid] = pmx; s_pk[1][wid] = pmn; }
    __syncthreads();
    pmx = s_pk[0][0]; pmn = s_pk[1][0];
#pragma unroll
    for (int q = 1; q < NW; ++q) { pmx = umax16x2(pmx, s_pk[0][q]); pmn = smin16x2_3(pmn, pmn, s_pk[1][q]); }
    uint32_t amax_pat = hmax_halves(pmx);
    // halves with bit 15 set saw a non-zero magnitude: (half & 0x7FFF) + 1 is the smallest one
    const uint32_t h0 = pmn & 0xFFFFu, h1 = pmn >> 16;
    uint32_t amin_pat = 0x7F7Fu;  // the reference starts amin at the bf16 maximum
    if (h0 & 0x8000u) amin_pat = min(amin_pat, (h0 & 0x7FFFu) + 1u);
    if (h1 & 0x8000u) amin_pat = min(amin_pat, (h1 & 0x7FFFu) + 1u);
    const bool has_nan = amax_pat > 0x7F80u;
    if (has_nan) {
        uint32_t mx = 0u, mn = 0x7F7Eu;
        auto scan = [&](uint32_t w) {
            const uint32_t lo = w & 0x7FFFu, hi = (w >> 16) & 0x7FFFu;
            const uint32_t lo_v = lo > 0x7F80u ? 0u : lo, hi_v = hi > 0x7F80u ? 0u : hi;
            mx = max(mx, max(lo_v, hi_v));
            mn = min(mn, min(lo_v - 1u, hi_v - 1u));
        };
#pragma unroll 1
        for (int n = 0; n < 16; ++n) {
            uint32_t w[VW];
            tile_unpack<VW>(chunk(n >> 2, n & 3), w);
#pragma unroll
            for (int q = 0; q < VW; ++q) scan(w[q]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
            mn = min(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, o));
        }
        __syncthreads();
        if (lane == 0) { s_pk[0][wid] = mx; s_pk[1][wid] = mn; }
        __syncthreads();
        amax_pat = s_pk[0][0]; amin_pat = s_pk[1][0];
#pragma unroll
        for (int q = 1; q < NW; ++q) { amax_pat = max(amax_pat, s_pk[0][q]); amin_pat = min(amin_pat, s_pk[1][q]); }
        amin_pat += 1u;
    }
    const float amax = u2f(amax_pat << 16), amin = u2f(amin_pat << 16);

    int repr = 0, code = 3, fmt = -1;
    if (qmode == QM_MOR) {
        repr = choose_by_range(amax, amin, clamp, dyn_mode != 0);
        if (repr == NEED_ERRORS) {
            ErrCtx<SF> e;
            e.s4 = __fdiv_rn(448.0f, amax);
            e.s5 = __fdiv_rn(57344.0f, amax);
            e.lut4 = s_lut4; e.lut5 = s_lut5;
            if constexpr (SF == kSfFp32) {
                fill_lut32t<kE4M3>(s_lut4, e.s4, tid, NT);
                fill_lut32t<kE5M2>(s_lut5, e.s5, tid, NT);
                __syncthreads();
            } else {
                e.c4 = e8_consts(e.s4);
                e.c5 = e8_consts(e.s5);
            }
            // every non-zero magnitude of the block lies in [amin, amax]
            const bool safe = bf16_div_safe(amin) && bf16_div_safe(amax);
            float a4[VW], a5[VW];
#pragma unroll
            for (int q = 0; q < VW; ++q) a4[q] = a5[q] = 0.0f;
            // The two errors of an element depend on its magnitude only (the casts are odd
            // functions), and a tile that reaches this pass spans at most 30 binades: they are
            // tabulated once per magnitude pattern in [amin, amax] (entry 0 = a zero element, no
            // error), and the 16384 elements look them up.  Same values, same order of additions.
            // Index i = pattern - (amin_pat - 1), so 1..n_pat are the magnitudes of the tile and 0 is
            // a zero element.  Within 2^13 of amax both casts work on normal numbers, even with a
            // power-of-two scale (x * scale > 224 * 2^-13 > 2^-6), and the errors repeat from one
            // binade to the next (x and 2x give q and 2q, the same quotient): rows of 128 indices
            // from row q_fold up share row q_fold's entries.
            const int n_pat = (int)(amax_pat - amin_pat) + 1;
            const int q_fold = max((n_pat >> 7) - 11, 1);
            const int n_tab = 128 * (q_fold + 1);          // entries 0 .. n_tab - 1
            // (the periodicity needs normal numbers throughout: a block whose amax is below 2^-96 could
            // meet denormal quotients q / scale in the folded rows, and takes the per-element form)
            if (!has_nan && n_tab <= table_entries && amax_pat >= 0x0F80u) {
                float2* tab = reinterpret_cast<float2*>(s_tile + kTileBytes);
                if (tid == 0) tab[0] = make_float2(0.0f, 0.0f);
                for (int i = 1 + 2 * tid; i < n_tab; i += 2 * NT) {  // two consecutive patterns per step
                    const uint32_t pl = amin_pat - 1u + (uint32_t)i;
                    const float lo = u2f(pl << 16), hi = u2f((pl + 1u) << 16);
                    float e4h, e4l, e5h, e5l;
                    if (safe) pair_errors<SF, true>(e, hi, lo, e4h, e4l, e5h, e5l);
                    else pair_errors<SF, false>(e, hi, lo, e4h, e4l, e5h, e5l);
                    tab[i] = make_float2(e4l, e5l);
                    if (i + 1 < n_tab) tab[i + 1] = make_float2(e4h, e5h);
                }
                __syncthreads();
                const int base = (int)amin_pat - 1, fold = q_fold << 7;
                if constexpr (RT) {
                    // Nearly every element of real data lies in the folded rows, whose 128 entries are indexed
                    // by the seven mantissa bits alone.  Sixteen copies of that row, interleaved so that lane r
                    // of a half-warp reads only bank pair r, make those lookups free of bank conflicts; they
                    // take the place of the tile's first 16 KiB (every thread holds its elements in registers).
                    // The few elements below the folded rows (and zeros) read the full table instead.
                    float2* rep = reinterpret_cast<float2*>(s_tile);
                    for (int i = tid; i < 2048; i += NT) rep[i] = tab[fold + (((i >> 4) - base) & 127)];
                    __syncthreads();
                    const uint32_t thr = (uint32_t)(base + fold);   // magnitude patterns from here up are folded
                    const uint32_t thr2 = thr * 0x00010001u;
                    const uint8_t* repl = s_tile + (tid & 15) * 8;
                    float2 acc2[VW];
#pragma unroll
                    for (int k = 0; k < VW; ++k) acc2[k] = make_float2(0.0f, 0.0f);
#pragma unroll
                    for (int n = 0; n < 16; ++n) {  // rows outer (j = n / 4), words inner (i = n % 4)
#pragma unroll
                        for (int k = 0; k < VW; ++k) {
                            const uint32_t w = tw[n][k];
                            float2 el = *reinterpret_cast<const float2*>(repl + ((w & 0x7Fu) << 7));
                            float2 eh = *reinterpret_cast<const float2*>(repl + ((w >> 9) & 0x3F80u));
                            if (umin16x2(mag2(w), thr2) != thr2) {   // rare: a half below the folded rows, or zero
                                const uint32_t ml = w & 0x7FFFu, mh = (w >> 16) & 0x7FFFu;
                                if (ml < thr) el = tab[max((int)ml - base, 0)];
                                if (mh < thr) eh = tab[max((int)mh - base, 0)];
                            }
                            // both formats' sums at once: packed binary32 additions, each half rounded on its own
                            acc2[k] = add_f32x2(acc2[k], add_f32x2(eh, el));
                        }
                    }
#pragma unroll
                    for (int k = 0; k < VW; ++k) { a4[k] = acc2[k].x; a5[k] = acc2[k].y; }
                } else {
#pragma unroll 2
                    for (int n = 0; n < 16; ++n) {  // rows outer (j = n / 4), words inner (i = n % 4)
                        uint32_t w[VW];
                        tile_unpack<VW>(chunk(n >> 2, n & 3), w);
#pragma unroll
                        for (int k = 0; k < VW; ++k) {
                            int il = max((int)(w[k] & 0x7FFFu) - base, 0), ih = max((int)((w[k] >> 16) & 0x7FFFu) - base, 0);
                            il = min(il, (il & 127) | fold);
                            ih = min(ih, (ih & 127) | fold);
                            const float2 el = tab[il], eh = tab[ih];
                            a4[k] = __fadd_rn(a4[k], __fadd_rn(eh.x, el.x));
                            a5[k] = __fadd_rn(a5[k], __fadd_rn(eh.y, el.y));
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int n = 0; n < 16; ++n) {  // rows outer (j = n / 4), words inner (i = n % 4)
                    uint32_t w[VW];
                    tile_unpack<VW>(chunk(n >> 2, n & 3), w);
#pragma unroll
                    for (int k = 0; k < VW; ++k) {
                        float e4, e5;
                        if (safe) word_errors_fast<SF, true>(e, bf16_hi(w[k]), bf16_lo(w[k]), e4, e5);
                        else word_errors_fast<SF, false>(e, bf16_hi(w[k]), bf16_lo(w[k]), e4, e5);
                        a4[k] = __fadd_rn(a4[k], e4);
                        a5[k] = __fadd_rn(a5[k], e5);
                    }
                }
            }
            const float w4 = logical_warp_sum<VW>(a4), w5 = logical_warp_sum<VW>(a5);
            if (tid % (32 / VW) == 0) { s_w4[tid / (32 / VW)] = w4; s_w5[tid / (32 / VW)] = w5; }
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

    V* dst = out + ((int64_t)by * 128) * cols_vec + (int64_t)bx * (4 * LPR);   // cols_vec in units of V
    auto store = [&](int n, const V& v) { st_stream(dst + (int64_t)(ty + 32 * (n >> 2)) * cols_vec + LPR * (n & 3) + a, v); };
    if (fmt < 0) {
        if constexpr (RT) {
#pragma unroll
            for (int n = 0; n < 16; ++n) store(n, tile_pack<VW>(tw[n]));
        } else {
#pragma unroll 4
            for (int n = 0; n < 16; ++n) store(n, chunk(n >> 2, n & 3));
        }
        return;
    }
    const float s = __fdiv_rn(fmt == kE2M3 ? 7.5f : (fmt == kE4M3 ? 448.0f : 57344.0f), amax);
    if constexpr (SF == kSfFp32) {
        if (fmt == kE4M3) fill_lut16<kE4M3>(s_lut16, s, tid, NT);
        else if (fmt == kE5M2) fill_lut16<kE5M2>(s_lut16, s, tid, NT);
        else fill_lut16<kE2M3>(s_lut16, s, tid, NT);
        __syncthreads();
        auto cast_all = [&](auto fmt_tag) {
            constexpr int F = decltype(fmt_tag)::value;
            if constexpr (RT) {
#pragma unroll
                for (int n = 0; n < 16; ++n) {
                    uint32_t w[VW];
#pragma unroll
                    for (int q = 0; q < VW; ++q) w[q] = lut_word<F>(s_lut16, tw[n][q], s);
                    store(n, tile_pack<VW>(w));
                }
            } else {
#pragma unroll 2
                for (int n = 0; n < 16; ++n) {
                    uint32_t w[VW];
                    tile_unpack<VW>(chunk(n >> 2, n & 3), w);
#pragma unroll
                    for (int q = 0; q < VW; ++q) w[q] = lut_word<F>(s_lut16, w[q], s);
                    store(n, tile_pack<VW>(w));
                }
            }
        };
        if (fmt == kE4M3) cast_all(std::integral_constant<int, kE4M3>{});
        else if (fmt == kE5M2) cast_all(std::integral_constant<int, kE5M2>{});
        else cast_all(std::integral_constant<int, kE2M3>{});
    } else {
        const E8Consts c = e8_consts(s);
        auto cast_all = [&](auto fmt_tag) {
            constexpr int F = decltype(fmt_tag)::value;
            if constexpr (RT) {
#pragma unroll
                for (int n = 0; n < 16; ++n) {
                    uint32_t w[VW];
#pragma unroll
                    for (int q = 0; q < VW; ++q) w[q] = e8_word<F>(tw[n][q], c);
                    store(n, tile_pack<VW>(w));
                }
            } else {
#pragma unroll 2
                for (int n = 0; n < 16; ++n) {
                    uint32_t w[VW];
                    tile_unpack<VW>(chunk(n >> 2, n & 3), w);
#pragma unroll
                    for (int q = 0; q < VW; ++q) w[q] = e8_word<F>(w[q], c);
                    store(n, tile_pack<VW>(w));
                }
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
    if (!is_fp32 && brows == 128 && bcols == 128 && rows % 128 == 0 && cols % 128 == 0 && aligned && !force_generic() &&
        rows < (int64_t(1) << 31) && cols < (int64_t(1) << 31)) {
        CUtensorMap map;
        if (make_tile_map(&map, in, rows, cols, 2, 32, 128)) {
            auto* o4 = static_cast<uint4*>(out);
            // the relative-error criterion keeps a table of (E4M3, E5M2) errors per magnitude pattern
            // behind the tile (at most 20 rows of 128 patterns after folding the periodic top rows) and
            // runs as 256 threads with 8-byte accesses, so that the four CTAs an SM can hold fill it
            const bool tabled = quant_mode == QM_MOR && !dynamic_range_mode;
            constexpr int kTabled = kTileBytes + kErrTableEntries * (int)sizeof(float2);
#define MORB_TILE(S)                                                                                                 \
    do {                                                                                                             \
        if (tabled) {                                                                                                \
            static SmemOptIn opt;                                                                                    \
            if (!opt(fq_tile128_kernel<S, 2>, kTabled)) return kErrLaunch;                                           \
            fq_tile128_kernel<S, 2><<<(unsigned)nb, 256, kTabled, st>>>(map, static_cast<uint2*>(out), meta, cols / 4, \
                                                                        (int)bx, clamp, quant_mode, dynamic_range_mode, \
                                                                        kErrTableEntries);                           \
        } else {                                                                                                     \
            fq_tile128_kernel<S, 4><<<(unsigned)nb, 128, kTileBytes, st>>>(map, static_cast<uint4*>(out), meta, cols / 8, \
                                                                           (int)bx, clamp, quant_mode, dynamic_range_mode, 0); \
        }                                                                                                            \
    } while (0)
            if (sf_type == kSfE8) MORB_TILE(kSfE8); else MORB_TILE(kSfFp32);
#undef MORB_TILE
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
