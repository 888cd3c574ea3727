// Single-pass fake-quantize with one scale per 1 x k group of a row: MX-style 1 x 32
// groups with power-of-two (E8M0) scales, per-row (per-channel) scaling, and anything
// between.  Semantics are those of quantize_kernel<BLOCK_SCALING_*> (ref: 801-823)
// with the element wrappers SQDD_{fp32,e8}_{e4m3,e5m2,e2m3} (ref: 356-379): group
// amax, scale = format max / amax (truncated to a power of two for E8 scaling),
// multiply, RNE cast, exact division, bf16 rounding.  An all-zero group is copied.
// One HBM read and one HBM write per element (4 bytes per bf16 element):
//   k <= 32 vectors : a group is a power-of-two set of lanes, amax by xor shuffles;
//   larger k        : one CTA per group, the group cached in registers between the
//                     amax pass and the cast, per-group look-up table for the
//                     division when the scale is a binary32 number.
// Instruction budget: at the HBM roofline a bf16 element has about 22 issue slots, so
// amax works on packed bf16 magnitudes (both halves of a word per instruction), the
// power-of-two scale is two float multiplies with its exponent taken from the amax
// bits (no division), and results of that path are packed without rounding (they are
// exact in bf16).
#include <cstdlib>
#include "kernels.cuh"
#include "tma.cuh"

namespace morb {

namespace {

// amax of a vector as a float; bf16 vectors go through packed integer maxima.  A NaN
// element makes the packed maximum exceed 0x7F80; the reference ignores NaNs (fmaxf),
// so that rare case is redone with float compares.
template <typename T>
__device__ __forceinline__ float vec_amax_float(const typename T::vec_t& v) {
    float a = 0.0f;
#pragma unroll
    for (int k = 0; k < T::kWordsPerVec; ++k) {
        float hi, lo;
        T::unpack(v, k, hi, lo);
        a = fmaxf(a, fmaxf(fabsf(hi), fabsf(lo)));
    }
    return a;
}
__device__ __forceinline__ uint32_t vec_amax_pattern(const uint4& v) {
    return hmax_halves(umax16x2_vec(mag2(v.x), mag2(v.y), mag2(v.z), mag2(v.w)));
}

template <typename T, int FMT, int SF>
__device__ __forceinline__ typename T::vec_t vec_cast_fp32scale(const typename T::vec_t& v, float s) {
    typename T::vec_t o;
#pragma unroll
    for (int k = 0; k < T::kWordsPerVec; ++k) {
        float hi, lo, rh, rl;
        T::unpack(v, k, hi, lo);
        sqdd_fp32_pair<FMT>(hi, lo, s, rh, rl);
        T::pack(o, k, rh, rl);
    }
    return o;
}

template <typename T, int FMT>
__device__ __forceinline__ typename T::vec_t vec_cast_e8(const typename T::vec_t& v, const E8Consts& c) {
    typename T::vec_t o;
#pragma unroll
    for (int k = 0; k < T::kWordsPerVec; ++k) {
        float hi, lo, rh, rl;
        T::unpack(v, k, hi, lo);
        sqdd_e8_pair_auto<FMT>(hi, lo, c, rh, rl);
        if constexpr (T::kBytesPerElem == 2) {
            // exact in bf16 (at most four significant bits) unless the literal path met a non-finite value
            const uint32_t w = c.fast ? pack_bf16_trunc(rh, rl) : pack_bf16(rh, rl);
            if (k == 0) o.x = w; else if (k == 1) o.y = w; else if (k == 2) o.z = w; else o.w = w;
        } else {
            T::pack(o, k, rh, rl);
        }
    }
    return o;
}

// scale constants of a group from its amax: the exponent comes from the amax bits when
// the quotient is a normal number, from the division itself otherwise
template <int FMT>
__device__ __forceinline__ E8Consts e8_from_amax(float a, float& scale_out) {
    const uint32_t ab = f2u(a);
    E8Consts c;
    int e8 = 1000;
    if ((ab >> 23) != 0u && (ab >> 23) != 0xFFu) e8 = e8_of_amax<FMT>(ab);
    if (e8_fast_ok(e8)) {
        c.e8 = e8; c.fast = true; c.up = pow2f(e8); c.down = pow2f(-e8);
        c.zero_bits = e8 < 0 ? ((uint32_t)(-e8) << 23) : 0u;
        scale_out = c.up;  // the E8M0 scale that is applied
    } else {
        const float s = __fdiv_rn(fmt_max<FMT>(), a);
        c = e8_consts(s);
        scale_out = u2f(f2u(s) & 0x7F800000u);
    }
    return c;
}

template <typename T, int FMT, int SF>
__global__ void __launch_bounds__(256)
group_small_kernel(const typename T::vec_t* __restrict__ in, typename T::vec_t* __restrict__ out,
                   float* __restrict__ scales, int64_t nvec, int lanes_per_group, int32_t* __restrict__ meta,
                   int64_t n_meta, int32_t meta_code) {
    const int64_t stride = (int64_t)gridDim.x * 256;
    const int64_t gtid = (int64_t)blockIdx.x * 256 + threadIdx.x;
    for (int64_t m = gtid; m < n_meta; m += stride) meta[m] = meta_code;
    constexpr int U = 4;
    // nvec is a multiple of 32, so whole warps enter or leave the loop together
    for (int64_t i = gtid; i < nvec; i += stride * U) {
        typename T::vec_t v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (i + u * stride < nvec) v[u] = ld_stream(in + i + u * stride);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (i + u * stride >= nvec) break;
            float a;
            if constexpr (T::kBytesPerElem == 2) {
                uint32_t p = vec_amax_pattern(v[u]);
                for (int o = lanes_per_group >> 1; o > 0; o >>= 1) p = max(p, __shfl_xor_sync(0xFFFFFFFFu, p, o));
                a = u2f(p << 16);
                if (__any_sync(0xFFFFFFFFu, p > 0x7F80u)) {  // a NaN in the warp: the reference's fmaxf skips it
                    a = vec_amax_float<T>(v[u]);
                    for (int o = lanes_per_group >> 1; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
                }
            } else {
                a = vec_amax_float<T>(v[u]);
                for (int o = lanes_per_group >> 1; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
            }
            float s = 1.0f;
            if (a > 0.0f) {
                if constexpr (SF == kSfE8) {
                    const E8Consts c = e8_from_amax<FMT>(a, s);
                    v[u] = vec_cast_e8<T, FMT>(v[u], c);
                } else {
                    s = __fdiv_rn(fmt_max<FMT>(), a);
                    v[u] = vec_cast_fp32scale<T, FMT, SF>(v[u], s);
                }
            }
            const int64_t idx = i + u * stride;
            st_stream(out + idx, v[u]);
            if (scales && (threadIdx.x & (lanes_per_group - 1)) == 0) scales[idx / lanes_per_group] = s;
        }
    }
}

// ---------------------------------------------------------------------------------
// bf16, power-of-two scale, groups of 1..32 vectors: the MX hot path
// ---------------------------------------------------------------------------------
// Everything a lane needs is derived from the packed amax pattern with integer
// operations; one warp-uniform test selects the branch-free body (normal finite amax,
// scale exponent inside the range where multiplying equals exponent-field
// arithmetic) and anything else (zero or non-finite group, extreme exponents) goes to
// the general code.
template <int FMT, bool NEG>
__device__ __forceinline__ uint4 mx_cast_vec(const uint4& v, float up, float down, uint32_t zero_bits) {
    uint4 o;
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t r[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float qh, ql;
        quant_dequant_pair<FMT, true>(__fmul_rn(bf16_hi(w[k]), up), __fmul_rn(bf16_lo(w[k]), up), qh, ql);
        float rh = __fmul_rn(qh, down), rl = __fmul_rn(ql, down);
        if constexpr (NEG) {  // a zero code under a scale below one comes back as +-2^(-e8-127)
            rh = qh == 0.0f ? u2f((f2u(qh) & 0x80000000u) | zero_bits) : rh;
            rl = ql == 0.0f ? u2f((f2u(ql) & 0x80000000u) | zero_bits) : rl;
        }
        r[k] = pack_bf16_trunc(rh, rl);
    }
    o.x = r[0]; o.y = r[1]; o.z = r[2]; o.w = r[3];
    return o;
}

// One 16-byte vector of a lane: group amax across the 2^GS lanes of the group, cast in
// place; returns the scale that was applied.  All 32 lanes call together.
template <int FMT, int GS>
__device__ __forceinline__ float mx_one(uint4& v) {
    constexpr int K127 = ((FMT == kE4M3) ? 8 : (FMT == kE5M2 ? 15 : 2)) + 127;
    constexpr uint32_t CMAN7 = (FMT == kE2M3) ? 0x70u : 0x60u;  // 1.875 / 1.75 as a 7-bit mantissa
    uint32_t p = vec_amax_pattern(v);
#pragma unroll
    for (int o = (1 << GS) >> 1; o > 0; o >>= 1) p = max(p, __shfl_xor_sync(0xFFFFFFFFu, p, o));
    const int ea = (int)(p >> 7);                               // exponent field of the group amax
    const int e8 = K127 - ea - ((p & 0x7Fu) > CMAN7 ? 1 : 0);   // exponent of RN(fmax / amax)
    const bool fast = (uint32_t)(ea - 1) < 254u && (uint32_t)(e8 + 119) <= 219u;
    float s;
    if (__all_sync(0xFFFFFFFFu, fast)) {
        const float up = u2f((uint32_t)(e8 + 127) << 23), down = u2f((uint32_t)(127 - e8) << 23);
        if (__any_sync(0xFFFFFFFFu, e8 < 0)) {
            const uint32_t zero_bits = e8 < 0 ? ((uint32_t)(-e8) << 23) : 0u;
            v = mx_cast_vec<FMT, true>(v, up, down, zero_bits);
        } else {
            v = mx_cast_vec<FMT, false>(v, up, down, 0u);
        }
        s = up;
    } else {
        float a = u2f(p << 16);
        if (__any_sync(0xFFFFFFFFu, p > 0x7F80u)) {  // a NaN in the warp: the reference's fmaxf skips it
            a = vec_amax_float<Bf16>(v);
#pragma unroll
            for (int o = (1 << GS) >> 1; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
        }
        s = 1.0f;
        if (a > 0.0f) v = vec_cast_e8<Bf16, FMT>(v, e8_from_amax<FMT>(a, s));
    }
    return s;
}

// Every warp streams its own 2 KiB chunks (four rows of 32 vectors) through a private
// two-stage shared-memory ring filled by bulk copies, so HBM reads stay in flight while
// the warp computes and no register holds data that has not arrived yet.  nvec is a
// multiple of 32: whole warps take every step together.
constexpr int kMxStages = 2, kMxChunkVec = 128, kMxWarps = 8;
template <int FMT, int GS>
__global__ void __launch_bounds__(32 * kMxWarps, 5)
mx_bf16_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, float* __restrict__ scales, int64_t nvec,
               int32_t* __restrict__ meta, int64_t n_meta, int32_t meta_code) {
    extern __shared__ __align__(128) uint8_t s_ring[];  // [warp][stage][2 KiB]
    __shared__ __align__(8) uint64_t s_bar[kMxWarps][kMxStages];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t n_warps = (int64_t)gridDim.x * kMxWarps, gw = (int64_t)blockIdx.x * kMxWarps + wid;
    WarpStream<kMxStages, kMxChunkVec * 16> ws;
    ws.start(s_ring + wid * (kMxStages * kMxChunkVec * 16), s_bar[wid], in, nvec * 16, gw, n_warps);
    for (int64_t m = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; m < n_meta; m += (int64_t)gridDim.x * blockDim.x)
        meta[m] = meta_code;
    const int64_t n_chunks = (nvec + kMxChunkVec - 1) / kMxChunkVec;
    const bool scale_lane = scales != nullptr && (lane & ((1 << GS) - 1)) == 0;
    int st = 0;
    for (int64_t c = gw; c < n_chunks; c += n_warps) {
        const int64_t v0 = c * kMxChunkVec;
        uint4* o = out + v0 + lane;
        float* sc = scales ? scales + ((v0 + lane) >> GS) : nullptr;
        const bool staged = ws.acquire(st);
        if (staged && v0 + kMxChunkVec <= nvec) {
            const uint4* chunk = reinterpret_cast<const uint4*>(ws.stage(st)) + lane;
#pragma unroll
            for (int r = 0; r < kMxChunkVec / 32; ++r) {
                uint4 v = chunk[r * 32];
                const float s = mx_one<FMT, GS>(v);
                st_stream(o + r * 32, v);
                if (scale_lane) sc[r * (32 >> GS)] = s;
            }
        } else {  // last, partial chunk, or a copy that did not arrive: ordinary loads
            const int nv = (int)(nvec - v0 < kMxChunkVec ? nvec - v0 : kMxChunkVec);
            for (int r = 0; r * 32 < nv; ++r) {
                uint4 v = ld_stream(in + v0 + r * 32 + lane);
                const float s = mx_one<FMT, GS>(v);
                st_stream(o + r * 32, v);
                if (scale_lane) sc[r * (32 >> GS)] = s;
            }
        }
        ws.release(st, c + kMxStages * n_warps);
        st = st + 1 == kMxStages ? 0 : st + 1;
    }
    ws.drain();
}

// ---------------------------------------------------------------------------------
// real quantized output: narrow-float codes + E8M0 scale bytes (no reference operator)
// ---------------------------------------------------------------------------------
// The codes are what the casts inside the power-of-two path produce before they are widened
// again (ref: 283-305, 356-379); the scale byte follows the MX convention, element =
// decode(code) * 2^(byte - 127).  Same stream structure and the same group amax as
// mx_bf16_kernel; 8 payload bytes per 16-byte input vector.
template <int FMT>
__device__ __forceinline__ uint32_t codes_fix_zero_sign(uint32_t c) {
    if constexpr (FMT == kE2M3 || FMT == kE3M2) {
        // the custom cast returns +0 for a zero result: drop bit 5 of a byte whose low five bits are zero
        const uint32_t nz = ((c & 0x1F1F1F1Fu) + 0x1F1F1F1Fu) & 0x20202020u;
        return c & (nz | 0x1F1F1F1Fu);
    } else {
        return c;
    }
}
template <int FMT, int GS>
__device__ __forceinline__ uint2 mx_codes_one(const uint4& v, uint32_t& scale_byte) {
    constexpr int K127 = ((FMT == kE4M3) ? 8 : (FMT == kE5M2 ? 15 : 2)) + 127;
    constexpr uint32_t CMAN7 = (FMT == kE2M3) ? 0x70u : 0x60u;
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t p = vec_amax_pattern(v);
#pragma unroll
    for (int o = (1 << GS) >> 1; o > 0; o >>= 1) p = max(p, __shfl_xor_sync(0xFFFFFFFFu, p, o));
    const int ea = (int)(p >> 7);
    int e8 = K127 - ea - ((p & 0x7Fu) > CMAN7 ? 1 : 0);
    const bool fast = (uint32_t)(ea - 1) < 254u && (uint32_t)(e8 + 119) <= 219u;
    uint32_t c[4];
    if (__all_sync(0xFFFFFFFFu, fast)) {
        const float up = u2f((uint32_t)(e8 + 127) << 23);
#pragma unroll
        for (int k = 0; k < 4; ++k) c[k] = cvt_codes<FMT>(__fmul_rn(bf16_hi(w[k]), up), __fmul_rn(bf16_lo(w[k]), up));
    } else {
        float a = u2f(p << 16);
        if (__any_sync(0xFFFFFFFFu, p > 0x7F80u)) {  // a NaN in the warp: the reference's fmaxf skips it
            a = vec_amax_float<Bf16>(v);
#pragma unroll
            for (int o = (1 << GS) >> 1; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
        }
        e8 = 0;
        if (a > 0.0f) e8 = e8_of_scale(__fdiv_rn(fmt_max<FMT>(), a));
#pragma unroll
        for (int k = 0; k < 4; ++k)
            c[k] = cvt_codes<FMT>(e8_shift_field(bf16_hi(w[k]), e8), e8_shift_field(bf16_lo(w[k]), e8));
    }
    scale_byte = (uint32_t)min(max(127 - e8, 0), 254);
    return make_uint2(codes_fix_zero_sign<FMT>(c[0] | (c[1] << 16)), codes_fix_zero_sign<FMT>(c[2] | (c[3] << 16)));
}

// eight codes of a vector: one byte each, or (PACK6) six bits each in 6 bytes, code i in bits
// [6 i, 6 i + 6) of the little-endian 48-bit group
template <bool PACK6>
__device__ __forceinline__ void store_codes(uint2* __restrict__ payload, int64_t idx, const uint2& c) {
    if constexpr (PACK6) {
        const uint32_t a = c.x, b = c.y;   // bytes c0..c3, c4..c7, each below 64
        const uint32_t lo = (a & 0x3Fu) | ((a >> 2) & 0xFC0u) | ((a >> 4) & 0x3F000u) | ((a >> 6) & 0xFC0000u) |
                            ((b & 0x3Fu) << 24) | ((b & 0x300u) << 22);
        const uint32_t hi = ((b >> 10) & 0xFu) | ((b >> 12) & 0x3F0u) | ((b >> 14) & 0xFC00u);
        uint16_t* p = reinterpret_cast<uint16_t*>(payload) + 3 * idx;
        p[0] = (uint16_t)lo; p[1] = (uint16_t)(lo >> 16); p[2] = (uint16_t)hi;
    } else {
        st_stream(payload + idx, c);
    }
}

template <int FMT, int GS, bool PACK6 = false>
__global__ void __launch_bounds__(32 * kMxWarps, 5)
mx_quantize_kernel(const uint4* __restrict__ in, uint2* __restrict__ payload, uint8_t* __restrict__ scales, int64_t nvec) {
    extern __shared__ __align__(128) uint8_t s_ring[];  // [warp][stage][2 KiB]
    __shared__ __align__(8) uint64_t s_bar[kMxWarps][kMxStages];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t n_warps = (int64_t)gridDim.x * kMxWarps, gw = (int64_t)blockIdx.x * kMxWarps + wid;
    WarpStream<kMxStages, kMxChunkVec * 16> ws;
    ws.start(s_ring + wid * (kMxStages * kMxChunkVec * 16), s_bar[wid], in, nvec * 16, gw, n_warps);
    const int64_t n_chunks = (nvec + kMxChunkVec - 1) / kMxChunkVec;
    const bool scale_lane = (lane & ((1 << GS) - 1)) == 0;
    int st = 0;
    for (int64_t c = gw; c < n_chunks; c += n_warps) {
        const int64_t v0 = c * kMxChunkVec;
        const int nv = (int)(nvec - v0 < kMxChunkVec ? nvec - v0 : kMxChunkVec);
        const bool staged = ws.acquire(st);
        const int64_t o = v0 + lane;
        uint8_t* sc = scales + ((v0 + lane) >> GS);
        if (staged && nv == kMxChunkVec) {
            const uint4* chunk = reinterpret_cast<const uint4*>(ws.stage(st)) + lane;
#pragma unroll
            for (int r = 0; r < kMxChunkVec / 32; ++r) {
                uint32_t sb;
                const uint2 codes = mx_codes_one<FMT, GS>(chunk[r * 32], sb);
                store_codes<PACK6>(payload, o + r * 32, codes);
                if (scale_lane) sc[r * (32 >> GS)] = (uint8_t)sb;
            }
        } else {  // last, partial chunk, or a copy that did not arrive: ordinary loads
            for (int r = 0; r * 32 < nv; ++r) {
                uint32_t sb;
                const uint2 codes = mx_codes_one<FMT, GS>(ld_stream(in + v0 + r * 32 + lane), sb);
                store_codes<PACK6>(payload, o + r * 32, codes);
                if (scale_lane) sc[r * (32 >> GS)] = (uint8_t)sb;
            }
        }
        ws.release(st, c + kMxStages * n_warps);
        st = st + 1 == kMxStages ? 0 : st + 1;
    }
    ws.drain();
}

constexpr int kRowThreads = 256;
constexpr int kRowMaxVec = 8;

// One CTA per group at a time, persistent over groups: while a group is reduced, cast
// and stored out of one register buffer, the loads of the CTA's next group are already
// in flight into the other, so every resident CTA always has HBM reads outstanding.
template <typename T, int FMT, int SF, int NV>
__global__ void __launch_bounds__(kRowThreads)
group_row_kernel(const typename T::vec_t* __restrict__ in, typename T::vec_t* __restrict__ out,
                 float* __restrict__ scales, int group_vec, int64_t n_groups, int32_t* __restrict__ meta,
                 int32_t meta_code) {
    __shared__ float s_red[2][kRowThreads / 32];
    __shared__ uint32_t s_lut[256];  // bf16 bits (bf16 output) or binary32 bits (binary32 output)
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    typename T::vec_t v[NV], nx[NV];
    auto load = [&](typename T::vec_t (&dst)[NV], int64_t g) {
        const typename T::vec_t* src = in + g * group_vec;
#pragma unroll
        for (int u = 0; u < NV; ++u)
            if (tid + u * kRowThreads < group_vec) dst[u] = ld_stream(src + tid + u * kRowThreads);
    };
    int64_t g = blockIdx.x;
    if (g < n_groups) load(v, g);
    for (int it = 0; g < n_groups; g += gridDim.x, ++it) {
        const int64_t gn = g + gridDim.x;
        if (gn < n_groups) load(nx, gn);
        float a = 0.0f;
        if constexpr (T::kBytesPerElem == 2) {
            uint32_t p = 0u;
#pragma unroll
            for (int u = 0; u < NV; ++u)
                if (tid + u * kRowThreads < group_vec) p = max(p, vec_amax_pattern(v[u]));
            a = u2f(p << 16);
            if (p > 0x7F80u) {
                a = 0.0f;
#pragma unroll
                for (int u = 0; u < NV; ++u)
                    if (tid + u * kRowThreads < group_vec) a = fmaxf(a, vec_amax_float<T>(v[u]));
            }
        } else {
#pragma unroll
            for (int u = 0; u < NV; ++u)
                if (tid + u * kRowThreads < group_vec) a = fmaxf(a, vec_amax_float<T>(v[u]));
        }
        a = warp_max(a);
        if (lane == 0) s_red[it & 1][wid] = a;
        __syncthreads();
#pragma unroll
        for (int w = 0; w < kRowThreads / 32; ++w) a = fmaxf(a, s_red[it & 1][w]);
        float s = 1.0f;
        if (a > 0.0f) {
            if constexpr (SF == kSfFp32) {
                s = __fdiv_rn(fmt_max<FMT>(), a);
                // result = f(code) for a fixed scale: tabulate with the exact division once
                constexpr int NCODES = (FMT == kE2M3) ? 64 : 256;
                for (int c = tid; c < NCODES; c += kRowThreads) {
                    float q = h_lo_to_f32(codes_to_h2<FMT>((uint32_t)c));
                    if (FMT == kE2M3 && q == 0.0f) q = 0.0f;
                    const float r = __fdiv_rn(q, s);
                    s_lut[c] = (T::kBytesPerElem == 2) ? f32_to_bf16_bits(r) : f2u(r);
                }
                __syncthreads();
#pragma unroll
                for (int u = 0; u < NV; ++u)
                    if (tid + u * kRowThreads < group_vec) {
#pragma unroll
                        for (int k = 0; k < T::kWordsPerVec; ++k) {
                            float hi, lo;
                            T::unpack(v[u], k, hi, lo);
                            const uint32_t c = cvt_codes<FMT>(__fmul_rn(hi, s), __fmul_rn(lo, s));
                            if constexpr (T::kBytesPerElem == 2) {
                                const uint32_t w = __byte_perm(s_lut[c & 0xFFu], s_lut[c >> 8], 0x5410);
                                if (k == 0) v[u].x = w; else if (k == 1) v[u].y = w; else if (k == 2) v[u].z = w; else v[u].w = w;
                            } else {
                                T::pack(v[u], k, u2f(s_lut[c >> 8]), u2f(s_lut[c & 0xFFu]));
                            }
                        }
                    }
            } else {
                const E8Consts c = e8_from_amax<FMT>(a, s);
#pragma unroll
                for (int u = 0; u < NV; ++u)
                    if (tid + u * kRowThreads < group_vec) v[u] = vec_cast_e8<T, FMT>(v[u], c);
            }
        }
        if (tid == 0) {
            if (meta) meta[g] = meta_code;
            if (scales) scales[g] = s;
        }
        typename T::vec_t* dst = out + g * group_vec;
#pragma unroll
        for (int u = 0; u < NV; ++u)
            if (tid + u * kRowThreads < group_vec) st_stream(dst + tid + u * kRowThreads, v[u]);
#pragma unroll
        for (int u = 0; u < NV; ++u) v[u] = nx[u];
        if constexpr (SF == kSfFp32) __syncthreads();  // the table is rewritten by the next group
    }
}

template <typename T, int FMT, int SF>
int launch_t(const void* in, void* out, float* scales, int32_t* meta, int32_t meta_code, int64_t rows, int64_t cols,
             int bcols, cudaStream_t st) {
    constexpr int EPV = 16 / T::kBytesPerElem;
    if (bcols % EPV || cols % bcols) return kErrUnsupportedShape;
    const int gvec = bcols / EPV;
    const int64_t nvec = rows * cols / EPV;
    const int64_t n_groups = rows * (cols / bcols);
    auto* i4 = static_cast<const typename T::vec_t*>(in);
    auto* o4 = static_cast<typename T::vec_t*>(out);
    if (gvec <= 32 && (gvec & (gvec - 1)) == 0 && nvec % 32 == 0) {
        int64_t grid = (nvec + 1023) / 1024;
        const int64_t cap = (int64_t)sm_count() * 8;
        if (grid > cap) grid = cap;
        if (grid < 1) grid = 1;
        if constexpr (T::kBytesPerElem == 2 && SF == kSfE8) {
            int shift = 0;
            while ((1 << shift) < gvec) ++shift;
            constexpr int kRing = kMxWarps * kMxStages * kMxChunkVec * 16;
            // The hardware's CTA scheduler evens out the speed differences between SMs only if
            // it has CTAs left to hand out: two chunks per warp (both requested as the warp
            // starts) measured best, a persistent grid with a static partition 20 % slower.
            constexpr int kChunksPerWarp = 2;
            const int64_t n_chunks = (nvec + kMxChunkVec - 1) / kMxChunkVec;
            int64_t g2 = (n_chunks + kMxWarps * kChunksPerWarp - 1) / (kMxWarps * kChunksPerWarp);
            if (g2 > 0x7FFFFFFF) return kErrTooLarge;
            if (g2 < 1) g2 = 1;
#define MORB_MX(GS)                                                                                                    \
    do {                                                                                                               \
        static SmemOptIn opt;                                                                                          \
        if (!opt(mx_bf16_kernel<FMT, GS>, kRing)) return kErrLaunch;                                                   \
        mx_bf16_kernel<FMT, GS><<<(unsigned)g2, 32 * kMxWarps, kRing, st>>>(i4, o4, scales, nvec, meta,               \
                                                                            meta ? n_groups : 0, meta_code);           \
    } while (0)
            switch (shift) {
                case 0: MORB_MX(0); break;
                case 1: MORB_MX(1); break;
                case 2: MORB_MX(2); break;
                case 3: MORB_MX(3); break;
                case 4: MORB_MX(4); break;
                default: MORB_MX(5); break;
            }
#undef MORB_MX
            return check_launch();
        }
        group_small_kernel<T, FMT, SF><<<(unsigned)grid, 256, 0, st>>>(i4, o4, scales, nvec, gvec, meta, meta ? n_groups : 0, meta_code);
        return check_launch();
    }
    if (gvec <= kRowThreads * kRowMaxVec) {
        int64_t grid = (n_groups + 1) / 2;  // two groups per CTA: the second one's loads overlap the first one's arithmetic
        if (grid > 0x7FFFFFFF) return kErrTooLarge;
        const int nv = (gvec + kRowThreads - 1) / kRowThreads;
#define MORB_ROW(NV) group_row_kernel<T, FMT, SF, NV><<<(unsigned)grid, kRowThreads, 0, st>>>(i4, o4, scales, gvec, n_groups, meta, meta_code)
        if (nv <= 1) MORB_ROW(1); else if (nv <= 2) MORB_ROW(2); else if (nv <= 4) MORB_ROW(4); else MORB_ROW(8);
#undef MORB_ROW
        return check_launch();
    }
    return kErrUnsupportedShape;
}

template <typename T>
int launch_fmt(const void* in, void* out, float* scales, int32_t* meta, int32_t meta_code, int64_t rows,
               int64_t cols, int bcols, int fmt, int sf, cudaStream_t st) {
#define MORB_GO(F) (sf == kSfE8 ? launch_t<T, F, kSfE8>(in, out, scales, meta, meta_code, rows, cols, bcols, st) \
                                : launch_t<T, F, kSfFp32>(in, out, scales, meta, meta_code, rows, cols, bcols, st))
    if (fmt == kE4M3) return MORB_GO(kE4M3);
    if (fmt == kE5M2) return MORB_GO(kE5M2);
    if (fmt == kE2M3) return MORB_GO(kE2M3);
#undef MORB_GO
    return kErrInvalidArgument;
}

}  // namespace

int launch_quantize_mx(const void* in, void* payload, uint8_t* scales, int64_t rows, int64_t cols, int bcols, int fmt,
                       int pack6, cudaStream_t st) {
    if (pack6 && fmt != kE2M3) return kErrInvalidArgument;
    if (bcols % 8 || cols % bcols) return kErrUnsupportedShape;
    const int gvec = bcols / 8;
    const int64_t nvec = rows * cols / 8;
    if (gvec > 32 || (gvec & (gvec - 1)) || nvec % 32) return kErrUnsupportedShape;
    int shift = 0;
    while ((1 << shift) < gvec) ++shift;
    constexpr int kRing = kMxWarps * kMxStages * kMxChunkVec * 16;
    constexpr int kChunksPerWarp = 2;
    const int64_t n_chunks = (nvec + kMxChunkVec - 1) / kMxChunkVec;
    int64_t grid = (n_chunks + kMxWarps * kChunksPerWarp - 1) / (kMxWarps * kChunksPerWarp);
    if (grid > 0x7FFFFFFF) return kErrTooLarge;
    if (grid < 1) grid = 1;
    auto* i4 = static_cast<const uint4*>(in);
    auto* p2 = static_cast<uint2*>(payload);
#define MORB_Q(F, GS)                                                                                                \
    do {                                                                                                             \
        static SmemOptIn opt;                                                                                        \
        if (!opt(mx_quantize_kernel<F, GS>, kRing)) return kErrLaunch;                                               \
        mx_quantize_kernel<F, GS><<<(unsigned)grid, 32 * kMxWarps, kRing, st>>>(i4, p2, scales, nvec);               \
    } while (0)
#define MORB_QS(F)                                                                                                   \
    do {                                                                                                             \
        switch (shift) {                                                                                             \
            case 0: MORB_Q(F, 0); break;                                                                             \
            case 1: MORB_Q(F, 1); break;                                                                             \
            case 2: MORB_Q(F, 2); break;                                                                             \
            case 3: MORB_Q(F, 3); break;                                                                             \
            case 4: MORB_Q(F, 4); break;                                                                             \
            default: MORB_Q(F, 5); break;                                                                            \
        }                                                                                                            \
    } while (0)
#define MORB_Q6(GS)                                                                                                  \
    do {                                                                                                             \
        static SmemOptIn opt;                                                                                        \
        if (!opt(mx_quantize_kernel<kE2M3, GS, true>, kRing)) return kErrLaunch;                                     \
        mx_quantize_kernel<kE2M3, GS, true><<<(unsigned)grid, 32 * kMxWarps, kRing, st>>>(i4, p2, scales, nvec);     \
    } while (0)
    if (pack6) {
        switch (shift) {
            case 0: MORB_Q6(0); break;
            case 1: MORB_Q6(1); break;
            case 2: MORB_Q6(2); break;
            case 3: MORB_Q6(3); break;
            case 4: MORB_Q6(4); break;
            default: MORB_Q6(5); break;
        }
    } else if (fmt == kE4M3) MORB_QS(kE4M3);
    else if (fmt == kE5M2) MORB_QS(kE5M2);
    else if (fmt == kE2M3) MORB_QS(kE2M3);
    else return kErrInvalidArgument;
#undef MORB_Q6
#undef MORB_QS
#undef MORB_Q
    return check_launch();
}

int launch_fq_group(const void* in, void* out, int is_fp32, float* scales, int32_t* meta, int32_t meta_code,
                    int64_t rows, int64_t cols, int bcols, int fmt, int sf_type, cudaStream_t st) {
    return is_fp32 ? launch_fmt<Fp32>(in, out, scales, meta, meta_code, rows, cols, bcols, fmt, sf_type, st)
                   : launch_fmt<Bf16>(in, out, scales, meta, meta_code, rows, cols, bcols, fmt, sf_type, st);
}

}  // namespace morb
