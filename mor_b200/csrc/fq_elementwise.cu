// Kernels whose scale is the same for the whole tensor (or absent): the
// CURRENT_SCALING modes of fake_quantize, the BF16 pass-through, the E8Mx cast and
// the binary32 test operators.  One HBM read and one HBM write per element,
// 16-byte accesses, persistent grid-stride loops sized to the SM count.
#include "kernels.cuh"
#include "e8mx_math.cuh"

namespace morb {

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

// Output of scale-cast-descale for a FIXED binary32 scale is a pure function of the
// narrow-float code, so each CTA tabulates it once with the exact IEEE division of
// the reference (ref: 310-316, 46-60) and the hot loop is multiply, cvt, table look-up.
template <int FMT>
__device__ __forceinline__ void build_lut_bf16(uint16_t* lut, float s) {
    for (int c = threadIdx.x; c < 256; c += blockDim.x) {
        const float q = h_lo_to_f32(codes_to_h2<FMT>((uint32_t)c));
        lut[c] = (uint16_t)f32_to_bf16_bits(__fdiv_rn(q, s));
    }
    __syncthreads();
}

template <int FMT, int SF>
__global__ void __launch_bounds__(kThreads) cast_uniform_bf16_kernel(const uint4* __restrict__ in,
                                                                     uint4* __restrict__ out, int64_t nvec,
                                                                     int64_t n_tail_words, float s,
                                                                     int32_t* __restrict__ meta, int64_t n_meta,
                                                                     int32_t meta_code) {
    __shared__ uint16_t lut[256];
    if constexpr (SF == kSfFp32) build_lut_bf16<FMT>(lut, s);
    const E8Consts e8c = e8_consts(s);
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t gtid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    for (int64_t m = gtid; m < n_meta; m += stride) meta[m] = meta_code;

    auto word = [&](uint32_t w) -> uint32_t {
        if constexpr (SF == kSfFp32) {
            const uint32_t c = cvt_codes<FMT>(__fmul_rn(bf16_hi(w), s), __fmul_rn(bf16_lo(w), s));
            return __byte_perm((uint32_t)lut[c & 0xFFu], (uint32_t)lut[c >> 8], 0x5410);
        } else {
            // the multiply form needs finite inputs; a caller-supplied scale comes with no amax
            // to vouch for them, so non-finite halves of the word take the literal form
            const bool finite = ((w & 0x7F80u) != 0x7F80u) && ((w & 0x7F800000u) != 0x7F800000u);
            float rh, rl;
            if (e8c.fast && finite) {
                sqdd_e8_pair_fast<FMT>(bf16_hi(w), bf16_lo(w), e8c.up, e8c.down, e8c.zero_bits, rh, rl);
                return pack_bf16_trunc(rh, rl);
            }
            sqdd_e8_pair<FMT>(bf16_hi(w), bf16_lo(w), e8c.e8, rh, rl);
            return pack_bf16(rh, rl);
        }
    };

    for (int64_t i = gtid; i < nvec; i += stride * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            if (i + u * stride < nvec) v[u] = ld_stream(in + i + u * stride);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            if (i + u * stride < nvec) {
                uint4 r;
                r.x = word(v[u].x); r.y = word(v[u].y); r.z = word(v[u].z); r.w = word(v[u].w);
                st_stream(out + i + u * stride, r);
            }
    }
    if (gtid < n_tail_words) {
        const uint32_t* tin = reinterpret_cast<const uint32_t*>(in + nvec);
        uint32_t* tout = reinterpret_cast<uint32_t*>(out + nvec);
        tout[gtid] = word(tin[gtid]);
    }
}

__global__ void __launch_bounds__(kThreads) copy_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                                        int64_t nvec, int64_t n_tail_bytes,
                                                        int32_t* __restrict__ meta, int64_t n_meta,
                                                        int32_t meta_code) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t gtid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    for (int64_t m = gtid; m < n_meta; m += stride) meta[m] = meta_code;
    if (in == out) return;
    for (int64_t i = gtid; i < nvec; i += stride * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            if (i + u * stride < nvec) v[u] = ld_stream(in + i + u * stride);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            if (i + u * stride < nvec) st_stream(out + i + u * stride, v[u]);
    }
    if (gtid < n_tail_bytes) {
        reinterpret_cast<uint8_t*>(out + nvec)[gtid] = reinterpret_cast<const uint8_t*>(in + nvec)[gtid];
    }
}

template <int FMT>
__global__ void __launch_bounds__(kThreads) quant_dequant_kernel(const float* __restrict__ in,
                                                                 float* __restrict__ out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride)
        out[i] = narrow_custom_fmt<FMT>(in[i]);
}

// ref: 865-875 + 248-306 with the custom E4M3 cast.  The per-element scale is
// 448.0 / x evaluated in double (the literal is a double) and narrowed to binary32.
template <bool RNE>
__global__ void __launch_bounds__(kThreads) e4m3_e8_scale_kernel(const float* __restrict__ in,
                                                                 float* __restrict__ out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        const float x = in[i];
        const float s = (float)__ddiv_rn(448.0, (double)x);
        const uint32_t sb = f2u(s), xb = f2u(x);
        int e8 = (int)((sb >> 23) & 0xFFu) - 127;
        const int xexp = (int)((xb >> 23) & 0xFFu);
        const uint32_t xman = xb & 0x7FFFFFu;
        if constexpr (RNE) {
            const uint32_t sman = sb & 0x7FFFFFu;
            const uint32_t guard = (sman >> 22) & 1u;
            const uint32_t sticky = (sman & ((1u << 22) - 1u)) != 0;
            // 6815744 = 0b1101 << 19: the largest mantissa that still rounds down to 1.75
            if (guard && xman <= 6815744u && xexp + e8 < 135 && (sticky | ((uint32_t)e8 & 1u))) e8 += 1;
        }
        const float q = narrow_custom_fmt<kE4M3>(e8_shift_field(x, e8));
        out[i] = e8_shift_field(q, -e8);
    }
}

template <int M>
__global__ void __launch_bounds__(kThreads) e8mx_cast_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                                             int64_t nvec, int64_t n_tail_words, int strategy,
                                                             const uint32_t* __restrict__ gamax_bits) {
    __shared__ uint32_t s_off[128];
    E8mxCast<M> cast;
    cast.init(s_off, e8mx_scale<M>(u2f(*gamax_bits), strategy), threadIdx.x);
    __syncthreads();
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t gtid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    for (int64_t i = gtid; i < nvec; i += stride * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            if (i + u * stride < nvec) v[u] = ld_stream(in + i + u * stride);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            if (i + u * stride < nvec) {
                uint4 r;
                r.x = cast.word(v[u].x); r.y = cast.word(v[u].y); r.z = cast.word(v[u].z); r.w = cast.word(v[u].w);
                st_stream(out + i + u * stride, r);
            }
    }
    if (gtid < n_tail_words) {
        const uint32_t* tin = reinterpret_cast<const uint32_t*>(in + nvec);
        uint32_t* tout = reinterpret_cast<uint32_t*>(out + nvec);
        tout[gtid] = cast.word(tin[gtid]);
    }
}

// ---- real quantized output under binary32 scales (no reference operator; get_scaling_factor ref: 1059-1093,
// the cast of SQDD_fp32_scale ref: 310-316) ----------------------------------------------------------
// ref: 1059-1093 for strategies 1, 3 and 4; the block amax is floored at 1e-35
__device__ __forceinline__ float payload_scale(int ss, float gamax, float bamax) {
    if (bamax < 1e-35f) bamax = 1e-35f;
    if (ss == 1) {
        const uint32_t gman = f2u(__fdiv_rn(448.0f, gamax)) & 0x007FFFFFu;
        const uint32_t bb = f2u(__fdiv_rn(448.0f, bamax));
        const float adj = u2f((bb & 0xFF800000u) | gman);
        return (gman <= (bb & 0x007FFFFFu)) ? adj : __fdiv_rn(adj, 2.0f);
    }
    if (ss == 3) return __fdiv_rn(448.0f, bamax);
    return gamax > 0.0f ? __fdiv_rn(448.0f, gamax) : 1.0f;
}
__global__ void __launch_bounds__(kThreads) block_scales_kernel(const float* __restrict__ block_amax, int64_t n_blocks, int ss,
                                                                const uint32_t* __restrict__ gamax_bits,
                                                                const float* __restrict__ ext_gamax,
                                                                float* __restrict__ scales, float* __restrict__ gamax_out) {
    const float gamax = ext_gamax ? *ext_gamax : u2f(*gamax_bits);
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i < n_blocks) scales[i] = payload_scale(ss, gamax, fabsf(block_amax[i]));   // the sign bit of a stored amax is a flag
    if (i == 0 && gamax_out) *gamax_out = gamax;
}
// E4M3 bytes of RN(x * scale), a zero element -> code 0.  A thread owns one 16-byte vector column and walks
// `rows_per_cta` consecutive rows, four loads in flight; its scale(s) change only when the walk enters the next
// row of blocks, so no index arithmetic is left per element.  The scale of an element is
// scales[(row / brows) * blocks_x + col / bcols]; a vector never straddles two blocks unless bcols == 1 (one
// scale per column), where the thread keeps one scale per element.
template <typename T>
__global__ void __launch_bounds__(kThreads) quantize_scaled_kernel(const typename T::vec_t* __restrict__ in,
                                                                   uint8_t* __restrict__ payload,
                                                                   const float* __restrict__ scales, int64_t rows,
                                                                   int cols_vec, int brows, int bcols, int blocks_x,
                                                                   int rows_per_cta) {
    constexpr int EPV = 16 / T::kBytesPerElem;
    const int cv = blockIdx.x * kThreads + threadIdx.x;
    if (cv >= cols_vec) return;
    const bool per_col = bcols == 1;
    const int bc = per_col ? cv * EPV : cv * EPV / bcols;
    int64_t r = (int64_t)blockIdx.y * rows_per_cta;
    const int64_t r_end = r + rows_per_cta < rows ? r + rows_per_cta : rows;
    int64_t br = r / brows;
    int rem = (int)(r - br * brows);
    float s[EPV];
    auto load_scales = [&]() {
        const float* p = scales + br * blocks_x + bc;
        const float first = __ldg(p);
#pragma unroll
        for (int j = 0; j < EPV; ++j) s[j] = per_col ? __ldg(p + j) : first;
    };
    load_scales();
    const typename T::vec_t* src = in + r * cols_vec + cv;
    uint8_t* dst = payload + (r * cols_vec + cv) * EPV;
    for (; r < r_end; r += 4) {
        typename T::vec_t v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (r + u < r_end) v[u] = ld_stream(src + (int64_t)u * cols_vec);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (r + u >= r_end) break;
            uint32_t codes[EPV / 2];
#pragma unroll
            for (int k = 0; k < T::kWordsPerVec; ++k) {
                float hi, lo;
                T::unpack(v[u], k, hi, lo);
                uint32_t c = cvt_codes<kE4M3>(__fmul_rn(hi, s[2 * k + 1]), __fmul_rn(lo, s[2 * k]));
                if (hi == 0.0f) c &= 0x00FFu;     // zeros (of either sign) are stored as +0
                if (lo == 0.0f) c &= 0xFF00u;
                codes[k] = c;                     // low byte: element 2k, high byte: element 2k + 1
            }
            uint8_t* d = dst + (int64_t)u * cols_vec * EPV;
            if constexpr (EPV == 8) {
                uint2 o;
                o.x = codes[0] | (codes[1] << 16);
                o.y = codes[2] | (codes[3] << 16);
                *reinterpret_cast<uint2*>(d) = o;
            } else {
                *reinterpret_cast<uint32_t*>(d) = codes[0] | (codes[1] << 16);
            }
            if (++rem == brows) {   // the next row belongs to the next row of blocks
                rem = 0;
                ++br;
                if (r + u + 1 < r_end) load_scales();
            }
        }
        src += (int64_t)4 * cols_vec;
        dst += (int64_t)4 * cols_vec * EPV;
    }
}

int grid_for(int64_t work_items_per_thread_unit) {
    // work_items = number of per-thread loop slots; at most 8 CTAs of 256 threads per SM
    const int64_t want = (work_items_per_thread_unit + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)sm_count() * 8;
    int64_t g = want < cap ? want : cap;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cached[dev] = n > 0 ? n : 148;
    }
    return cached[dev];
}

int check_launch() { return cudaGetLastError() == cudaSuccess ? kOk : kErrLaunch; }

namespace { int g_kernel_selection = 0; }
bool force_generic() { return (g_kernel_selection & 1) != 0; }
bool resident_disabled() { return (g_kernel_selection & 2) != 0; }
void set_kernel_selection(int mask) { g_kernel_selection = mask; }

int launch_cast_uniform(const void* in, void* out, int64_t n_elems, int fmt, int sf_type, float scale,
                        int32_t* meta, int64_t n_meta, int32_t meta_code, cudaStream_t st) {
    const int64_t nvec = n_elems / 8;
    const int64_t tail_words = (n_elems % 8) / 2;
    const int g = grid_for(nvec > n_meta ? nvec : n_meta);
    auto* i4 = static_cast<const uint4*>(in);
    auto* o4 = static_cast<uint4*>(out);
#define MORB_GO(F, S) cast_uniform_bf16_kernel<F, S><<<g, kThreads, 0, st>>>(i4, o4, nvec, tail_words, scale, meta, n_meta, meta_code)
    if (fmt == kE4M3 && sf_type == kSfFp32) MORB_GO(kE4M3, kSfFp32);
    else if (fmt == kE4M3 && sf_type == kSfE8) MORB_GO(kE4M3, kSfE8);
    else if (fmt == kE5M2 && sf_type == kSfFp32) MORB_GO(kE5M2, kSfFp32);
    else if (fmt == kE5M2 && sf_type == kSfE8) MORB_GO(kE5M2, kSfE8);
    else return kErrInvalidArgument;
#undef MORB_GO
    return check_launch();
}

int launch_copy(const void* in, void* out, int64_t n_bytes, int32_t* meta, int64_t n_meta, int32_t meta_code,
                cudaStream_t st) {
    const int64_t nvec = n_bytes / 16;
    const int g = grid_for(nvec > n_meta ? nvec : n_meta);
    copy_kernel<<<g, kThreads, 0, st>>>(static_cast<const uint4*>(in), static_cast<uint4*>(out), nvec, n_bytes % 16,
                                        meta, n_meta, meta_code);
    return check_launch();
}

int launch_quantize_scaled(const void* in, int is_fp32, uint8_t* payload, float* scales, float* gamax_out, int64_t rows,
                           int64_t cols, int brows, int bcols, int ss, const float* block_amax, int64_t n_blocks,
                           const uint32_t* gamax_bits, const float* ext_gamax, cudaStream_t st) {
    block_scales_kernel<<<(unsigned)((n_blocks + kThreads - 1) / kThreads), kThreads, 0, st>>>(block_amax, n_blocks, ss, gamax_bits,
                                                                                                ext_gamax, scales, gamax_out);
    int rc = check_launch();
    if (rc) return rc;
    const int epv = is_fp32 ? 4 : 8;
    const int64_t cols_vec = cols / epv, blocks_x = cols / bcols;
    if (cols_vec >= (int64_t(1) << 31) || blocks_x >= (int64_t(1) << 31)) return kErrTooLarge;
    int64_t rpc = 16;                                     // rows per CTA; grid.y is limited to 65535
    if ((rows + rpc - 1) / rpc > 65535) rpc = (rows + 65534) / 65535;
    if (rpc >= (int64_t(1) << 31)) return kErrTooLarge;
    const dim3 grid((unsigned)((cols_vec + kThreads - 1) / kThreads), (unsigned)((rows + rpc - 1) / rpc));
    if (is_fp32) quantize_scaled_kernel<Fp32><<<grid, kThreads, 0, st>>>(static_cast<const float4*>(in), payload, scales, rows, (int)cols_vec, brows, bcols, (int)blocks_x, (int)rpc);
    else quantize_scaled_kernel<Bf16><<<grid, kThreads, 0, st>>>(static_cast<const uint4*>(in), payload, scales, rows, (int)cols_vec, brows, bcols, (int)blocks_x, (int)rpc);
    return check_launch();
}

int launch_quant_dequant(const float* in, float* out, int64_t n, int fmt, cudaStream_t st) {
    const int g = grid_for(n);
    switch (fmt) {
        case kE4M3: quant_dequant_kernel<kE4M3><<<g, kThreads, 0, st>>>(in, out, n); break;
        case kE5M2: quant_dequant_kernel<kE5M2><<<g, kThreads, 0, st>>>(in, out, n); break;
        case kE3M2: quant_dequant_kernel<kE3M2><<<g, kThreads, 0, st>>>(in, out, n); break;
        case kE2M3: quant_dequant_kernel<kE2M3><<<g, kThreads, 0, st>>>(in, out, n); break;
        default: return kErrInvalidArgument;
    }
    return check_launch();
}

int launch_e4m3_e8_scale(const float* in, float* out, int64_t n, int rne, cudaStream_t st) {
    const int g = grid_for(n);
    if (rne) e4m3_e8_scale_kernel<true><<<g, kThreads, 0, st>>>(in, out, n);
    else e4m3_e8_scale_kernel<false><<<g, kThreads, 0, st>>>(in, out, n);
    return check_launch();
}

int launch_e8mx_cast(const void* in, void* out, int64_t n_elems, int qtype, int strategy,
                     const uint32_t* gamax_bits, cudaStream_t st) {
    const int64_t nvec = n_elems / 8;
    const int64_t tail_words = (n_elems % 8) / 2;
    const int g = grid_for(nvec);
    auto* i4 = static_cast<const uint4*>(in);
    auto* o4 = static_cast<uint4*>(out);
    switch (qtype) {
        case 1: e8mx_cast_kernel<1><<<g, kThreads, 0, st>>>(i4, o4, nvec, tail_words, strategy, gamax_bits); break;
        case 2: e8mx_cast_kernel<2><<<g, kThreads, 0, st>>>(i4, o4, nvec, tail_words, strategy, gamax_bits); break;
        case 3: e8mx_cast_kernel<3><<<g, kThreads, 0, st>>>(i4, o4, nvec, tail_words, strategy, gamax_bits); break;
        default: return kErrInvalidArgument;
    }
    return check_launch();
}

}  // namespace morb
