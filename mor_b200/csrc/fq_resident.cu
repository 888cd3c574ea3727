// fake_quantize_block_scaling on 128 x 128 blocks as ONE kernel, for tensors small enough to
// stay in the shared memories of the GPU between the two passes (ref: the five launches at
// fake_quantize.cu:2093-2099; the reference authors' cooperative prototype is
// jatin/fake_quantize_num_blocks.cu:973-1233).
//
// One CTA of 1024 threads per SM, launched cooperatively so that every CTA is resident.  A CTA
// owns up to kSlots tiles (7 of bf16, 3 of binary32) and requests all of them by TMA as it
// starts: the tensor is read from HBM exactly once.
//
//   pass 1   per tile, as it arrives: amax, non-zero count and the screening flags of the short
//            quotient, from shared memory; one atomicMax / atomicAdd per CTA for the tensor.
//   barrier  every CTA now knows the tensor's amax.
//   pass 2   per tile: scale (ref: 1059-1093), table of quotients, E4M3 cast, store, error sum
//            in the reference's order (ref: 1117-1156): thread (tx, ty) of the 32 x 32 CTA is a
//            real thread here, rows ty + 32 j outer, words tx + 32 i inner, high half first.
//   barrier  every CTA now sees every block's error sum.
//   decide   every CTA repeats the reference's ordered sum (thread t adds entries t, t + 1024;
//            ref: 1183-1196) -- same additions, same bits -- and, if the tensor stays BF16
//            (ref: 1203-1241), writes its tiles back from shared memory.  The input is never
//            read again, so output == input needs no special order.
//
// The two grid barriers are counters in the workspace head (zeroed by the launch before this
// one); every wait -- barrier or TMA -- is bounded, and a wait that runs out is reported as
// meta = -1 instead of hanging the GPU.
#include <type_traits>

#include "kernels.cuh"
#include "scaling_math.cuh"
#include "tma.cuh"

namespace morb {

namespace {

constexpr int kResThreads = 1024;

template <typename T> struct Res {
    static constexpr int kTileBytes = 128 * 128 * T::kBytesPerElem;
    static constexpr int kSlots = T::kBytesPerElem == 2 ? 7 : 3;
    // behind the tiles: mbarriers, per-tile statistics, warp sums, two quotient tables
    static constexpr int kBarOff = kSlots * kTileBytes;   // 8 x uint64
    static constexpr int kAmaxOff = kBarOff + 64;          // 8 x uint32  tile amax bits
    static constexpr int kNnzOff = kAmaxOff + 32;          // 8 x int32   tile non-zero count
    static constexpr int kFlagOff = kNnzOff + 32;          // 8 x uint32  bit 0: short quotient not allowed, bit 1: NaN seen
    static constexpr int kWsumOff = kFlagOff + 32;         // 32 x float
    static constexpr int kMiscOff = kWsumOff + 128;        // 8 x uint32
    static constexpr int kLutOff = kMiscOff + 32;          // 2 x 256 x float
    static constexpr int kSmem = kLutOff + 2 * 1024;
    static_assert(kLutOff % 16 == 0, "table alignment");
    static_assert(kSmem <= 227 * 1024, "shared memory of one SM");
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All CTAs of the (cooperative) grid meet here.  False for every thread of the CTA if the
// others did not show up within the limit.
__device__ __forceinline__ bool grid_barrier(uint32_t* counter, uint32_t expected, uint32_t limit) {
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
        uint32_t polls = 0;
        while (ld_acquire_gpu(counter) < expected) {
            if (++polls > limit) { ok = false; break; }
        }
        __threadfence();
    }
    return __syncthreads_and(ok) != 0;
}

// word = the pair of elements (2w, 2w + 1): 4 bytes of bf16, 8 bytes of binary32
template <typename T> struct Word;
template <> struct Word<Bf16> {
    using type = uint32_t;
    __device__ static __forceinline__ void unpack(uint32_t w, float& hi, float& lo) { hi = bf16_hi(w); lo = bf16_lo(w); }
};
template <> struct Word<Fp32> {
    using type = float2;
    __device__ static __forceinline__ void unpack(float2 w, float& hi, float& lo) { hi = w.y; lo = w.x; }
};

// pass 2 of one tile: thread (tx, ty) walks its eight words in the reference's order
template <typename T, int DIV, bool NOZERO, typename P>
__device__ __forceinline__ float cast_tile(const P& path, const uint8_t* tile, typename Word<T>::type* dst, int64_t cols_w,
                                           int tx, int ty) {
    using W = typename Word<T>::type;
    const W* t = reinterpret_cast<const W*>(tile);
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = ty + 32 * j, c = tx + 32 * i;
            float hi, lo, dh, dl, eh, el;
            Word<T>::unpack(t[r * 64 + c], hi, lo);
            err_pair<DIV, P, NOZERO>(path, hi, lo, dh, dl, eh, el);
            acc = __fadd_rn(acc, eh);
            acc = __fadd_rn(acc, el);
            if constexpr (T::kBytesPerElem == 2) {
                uint32_t w;
                if constexpr (PathTraits<P>::kExactBf16) w = path.c.fast ? pack_bf16_trunc(dh, dl) : pack_bf16(dh, dl);
                else w = pack_bf16_round(dh, dl);
                __stcs(dst + (int64_t)r * cols_w + c, w);
            } else {
                __stcs(dst + (int64_t)r * cols_w + c, make_float2(dl, dh));
            }
        }
    }
    return acc;
}

template <typename T, bool E8>
__global__ void __launch_bounds__(kResThreads, 1)
block_resident_kernel(const __grid_constant__ CUtensorMap tmap, void* __restrict__ out_raw, int64_t cols, int blocks_x,
                      int n_tiles, int ss, float threshold, float* __restrict__ block_err, ScalarsWs* __restrict__ ws,
                      int32_t* __restrict__ meta_out, float* __restrict__ gamax_out, void* __restrict__ gnnz_out,
                      int nnz_is_i64, float* __restrict__ gerr_out, uint32_t spin_limit) {
    using R = Res<T>;
    using W = typename Word<T>::type;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + R::kBarOff);
    uint32_t* s_amax = reinterpret_cast<uint32_t*>(smem + R::kAmaxOff);
    int* s_nnz = reinterpret_cast<int*>(smem + R::kNnzOff);
    uint32_t* s_flag = reinterpret_cast<uint32_t*>(smem + R::kFlagOff);
    float* s_wsum = reinterpret_cast<float*>(smem + R::kWsumOff);
    uint32_t* s_misc = reinterpret_cast<uint32_t*>(smem + R::kMiscOff);
    float* s_lut = reinterpret_cast<float*>(smem + R::kLutOff);

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int G = gridDim.x;
    // this CTA's tiles: blockIdx.x, blockIdx.x + G, ...
    const int n_mine = (n_tiles - (int)blockIdx.x + G - 1) / G;   // 1 .. kSlots (the launcher guarantees it)

    if (tid == 0) {
        for (int k = 0; k < R::kSlots; ++k) mbar_init(&s_bar[k], 1);
    }
    if (tid < 8) { s_amax[tid] = 0u; s_nnz[tid] = 0; s_flag[tid] = 0u; }
    __syncthreads();
    if (lane == 0 && wid < n_mine) {
        const int t = (int)blockIdx.x + wid * G;
        mbar_expect_tx(&s_bar[wid], R::kTileBytes);
        tma_load_2d(smem + wid * R::kTileBytes, &tmap, (t % blocks_x) * 128, (t / blocks_x) * 128, &s_bar[wid]);
    }

    // ---- pass 1: statistics of every tile, as it arrives --------------------------------
    bool arrived = true;
    for (int k = 0; k < n_mine; ++k) {
        if (!__all_sync(0xFFFFFFFFu, mbar_wait_bounded(&s_bar[k], 0))) { arrived = false; break; }   // warp-uniform
        const uint8_t* tile = smem + k * R::kTileBytes;
        uint32_t amax_bits, flags = 0u;
        int nnz = 0;
        if constexpr (T::kBytesPerElem == 2) {
            const uint4* tv = reinterpret_cast<const uint4*>(tile);
            uint32_t pmx = 0u, pmn = 0x7FFF7FFFu;
            int nnz4 = 0;
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const uint4 v = tv[tid + u * kResThreads];
                const uint32_t m0 = mag2(v.x), m1 = mag2(v.y), m2 = mag2(v.z), m3 = mag2(v.w);
                pmx = umax16x2_3(umax16x2_3(pmx, m0, m1), m2, m3);
                const uint32_t s0 = m0 + 0x7FFF7FFFu, s1 = m1 + 0x7FFF7FFFu, s2 = m2 + 0x7FFF7FFFu, s3 = m3 + 0x7FFF7FFFu;
                pmn = smin16x2_3(smin16x2_3(pmn, s0, s1), s2, s3);
                nnz4 += __popc((top_bits_to_bytes(s0, s1) & 0x0F0F0F0Fu) | (top_bits_to_bytes(s2, s3) & 0xF0F0F0F0u));
            }
            nnz = nnz4 >> 2;
            const uint32_t top = hmax_halves(pmx);
            amax_bits = top << 16;
            // smallest non-zero magnitude this thread saw (a half with bit 15 set saw one)
            const uint32_t h0 = pmn & 0xFFFFu, h1 = pmn >> 16;
            uint32_t amin_pat = 0x3F80u;
            if (h0 & 0x8000u) amin_pat = min(amin_pat, (h0 & 0x7FFFu) + 1u);
            if (h1 & 0x8000u) amin_pat = min(amin_pat, (h1 & 0x7FFFu) + 1u);
            if (top > 0x7F80u) flags |= 3u;                                            // NaN: exact rescan below
            if (!bf16_div_safe(u2f(amin_pat << 16)) || (top != 0u && !bf16_div_safe(u2f(top << 16)))) flags |= 1u;
        } else {
            const float4* tv = reinterpret_cast<const float4*>(tile);
            float a = 0.0f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float4 v = tv[tid + u * kResThreads];
                const float a0 = fabsf(v.x), a1 = fabsf(v.y), a2 = fabsf(v.z), a3 = fabsf(v.w);
                a = fmaxf(a, fmaxf(fmaxf(a0, a1), fmaxf(a2, a3)));   // fmaxf skips NaNs, as the reference's does
                nnz += (a0 > 0.0f) + (a1 > 0.0f) + (a2 > 0.0f) + (a3 > 0.0f);
            }
            amax_bits = f2u(a);
        }
        amax_bits = __reduce_max_sync(0xFFFFFFFFu, amax_bits);
        nnz = __reduce_add_sync(0xFFFFFFFFu, nnz);
        flags = __reduce_or_sync(0xFFFFFFFFu, flags);
        if (lane == 0) {
            atomicMax(&s_amax[k], amax_bits);
            if (nnz) atomicAdd(&s_nnz[k], nnz);
            if (flags) atomicOr(&s_flag[k], flags);
        }
    }
    arrived = __syncthreads_and(arrived) != 0;
    if constexpr (T::kBytesPerElem == 2) {
        // a NaN in a tile: the packed maximum is not the reference's (fmaxf ignores NaNs and they are
        // not counted); redo that tile with float compares
        for (int k = 0; k < n_mine && arrived; ++k) {
            if (!(s_flag[k] & 2u)) continue;      // CTA-uniform
            __syncthreads();
            if (tid == 0) { s_amax[k] = 0u; s_nnz[k] = 0; }
            __syncthreads();
            const uint4* tv = reinterpret_cast<const uint4*>(smem + k * R::kTileBytes);
            float a = 0.0f;
            int n = 0;
            for (int u = 0; u < 2; ++u) {
                const uint4 v = tv[tid + u * kResThreads];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float hi, lo;
                    Bf16::unpack(v, q, hi, lo);
                    const float ah = fabsf(hi), al = fabsf(lo);
                    a = fmaxf(a, fmaxf(ah, al));
                    n += (ah > 0.0f) + (al > 0.0f);
                }
            }
            a = warp_max(a);
            n = warp_sum_int(n);
            if (lane == 0) { atomicMax(&s_amax[k], f2u(a)); if (n) atomicAdd(&s_nnz[k], n); }
            __syncthreads();
        }
    }
    if (tid == 0) {
        uint32_t a = 0u;
        long long n = 0;
        for (int k = 0; k < n_mine; ++k) { a = max(a, s_amax[k]); n += s_nnz[k]; }
        if (arrived) {
            atomicMax(&ws->gamax_bits, a);
            if (n) atomicAdd(&ws->gnnz, (unsigned long long)n);
        } else {
            atomicOr(&ws->load_timeout, 1u);
        }
    }
    bool alive = grid_barrier(&ws->bar[0], (uint32_t)G, spin_limit);
    // a CTA whose tile did not arrive told the others before the barrier: everybody stops here
    alive = alive && *reinterpret_cast<volatile uint32_t*>(&ws->load_timeout) == 0u;
    if (!alive) {
        if (tid == 0) {
            atomicOr(&ws->load_timeout, 1u);
            if (blockIdx.x == 0 && meta_out) *meta_out = -1;
        }
        // give copies that may still be in flight a last bounded chance before the shared memory is released
        for (int k = 0; k < n_mine; ++k) mbar_wait_bounded(&s_bar[k], 0);
        return;
    }

    // ---- pass 2: scale, cast, store, error sums ---------------------------------------
    const float gamax = u2f(*reinterpret_cast<volatile uint32_t*>(&ws->gamax_bits));
    W* out = static_cast<W*>(out_raw);
    const int64_t cols_w = cols / 2;
    const int tx = lane, ty = wid;
    for (int k = 0; k < n_mine; ++k) {
        const int t = (int)blockIdx.x + k * G;
        const int bx = t % blocks_x, by = t / blocks_x;
        const uint8_t* tile = smem + k * R::kTileBytes;
        const float bamax = u2f(s_amax[k]);
        const bool zero_free = s_nnz[k] == 128 * 128 && !(s_flag[k] & 2u);
        const bool short_ok = T::kBytesPerElem != 2 || !(s_flag[k] & 1u);
        const float sf = scaling_factor(ss, gamax, bamax);
        W* dst = out + (int64_t)by * 128 * cols_w + (int64_t)bx * 64;
        float acc;
        auto dispatch = [&](const auto& path) {
            using P = std::decay_t<decltype(path)>;
            constexpr int kShort = T::kBytesPerElem == 2 ? kDivBf16 : kDivIeee;
            constexpr int kLong = T::kBytesPerElem == 2 ? kDivBf16Any : kDivIeee;
            if (short_ok && zero_free) acc = cast_tile<T, kShort, true, P>(path, tile, dst, cols_w, tx, ty);
            else if (short_ok) acc = cast_tile<T, kShort, false, P>(path, tile, dst, cols_w, tx, ty);
            else acc = cast_tile<T, kLong, false, P>(path, tile, dst, cols_w, tx, ty);
        };
        if constexpr (E8) {
            dispatch(PathE8{e8_consts(sf)});
        } else {
            float* lut = s_lut + (k & 1) * 256;
            // the table depends on the scale only: under the tensor-wide scale (ss_mode 4) it is filled once
            if (k == 0 || ss != 4) {
                fill_lut32(lut, sf, tid, kResThreads);
                __syncthreads();
            } else {
                lut = s_lut;
            }
            dispatch(PathLut{lut, sf});
        }
        const float s = warp_sum_ordered(acc);
        if (lane == 0) s_wsum[wid] = s;
        __syncthreads();
        if (wid == 0) {
            const float tot = warp_sum_ordered(s_wsum[lane]);
            if (lane == 0) block_err[t] = tot;
        }
        if (E8 || ss == 4) __syncthreads();   // no table barrier in the next round: keep s_wsum until warp 0 has read it
    }
    if (!grid_barrier(&ws->bar[1], (uint32_t)G, spin_limit)) {
        if (tid == 0) {
            atomicOr(&ws->load_timeout, 1u);
            if (blockIdx.x == 0 && meta_out) *meta_out = -1;
        }
        return;
    }

    // ---- decision: every CTA repeats the ordered sum of all blocks' errors -------------
    float acc = 0.0f;
    for (int e = tid; e < n_tiles; e += kResThreads) acc = __fadd_rn(acc, __ldcg(block_err + e));
    acc = warp_sum_ordered(acc);
    __syncthreads();
    if (lane == 0) s_wsum[wid] = acc;
    __syncthreads();
    if (wid == 0) {
        const float total = warp_sum_ordered(s_wsum[lane]);
        if (lane == 0) {
            const long long nnz = (long long)*reinterpret_cast<volatile unsigned long long*>(&ws->gnnz);
            const float avg = __fdiv_rn(total, (float)nnz);
            const int fb = avg > threshold;
            s_misc[0] = (uint32_t)fb;
            if (blockIdx.x == 0) {
                ws->fallback = fb;
                ws->gerr = total;
                ws->meta = fb ? 3 : 1;
                if (meta_out) *meta_out = fb ? 3 : 1;
                if (gamax_out) *gamax_out = gamax;
                if (gerr_out) *gerr_out = total;
                if (gnnz_out) {
                    if (nnz_is_i64) *static_cast<long long*>(gnnz_out) = nnz;
                    else *static_cast<int32_t*>(gnnz_out) = (int32_t)nnz;
                }
            }
        }
    }
    __syncthreads();
    if (s_misc[0]) {
        // the tensor stays as it was: the tiles are still in shared memory
        constexpr int kVecPerRow = 128 * T::kBytesPerElem / 16;
        const int64_t cols_v = cols * T::kBytesPerElem / 16;
        uint4* out_v = static_cast<uint4*>(out_raw);
        for (int k = 0; k < n_mine; ++k) {
            const int t = (int)blockIdx.x + k * G;
            const int bx = t % blocks_x, by = t / blocks_x;
            const uint4* tv = reinterpret_cast<const uint4*>(smem + k * R::kTileBytes);
            for (int v = tid; v < 128 * kVecPerRow; v += kResThreads) {
                const int r = v / kVecPerRow, c = v % kVecPerRow;
                __stcs(out_v + ((int64_t)by * 128 + r) * cols_v + (int64_t)bx * kVecPerRow + c, tv[v]);
            }
        }
    }
}

// box of one whole 128 x 128 tile (row-major in shared memory)
bool make_whole_tile_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int elem_bytes) {
    return make_tile_map(map, base, rows, cols, elem_bytes, 128, 128);
}

struct DeviceCaps {
    int checked = 0;   // 0 not yet, 1 usable, -1 not usable
    int ctas = 0;      // co-resident CTAs of the kernel on the device
};

template <typename T, bool E8>
int launch_resident_t(const ScalingArgs& a, int32_t* meta, float* gamax, void* gnnz, int nnz64, float* gerr,
                      cudaStream_t st) {
    using R = Res<T>;
    const int64_t bx = a.cols / 128, nt64 = bx * (a.rows / 128);
    static DeviceCaps caps[64];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kErrUnsupportedShape;
    DeviceCaps& c = caps[dev];
    auto kernel = block_resident_kernel<T, E8>;
    if (c.checked == 0) {
        int coop = 0, per_sm = 0;
        static SmemOptIn opt;
        if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) == cudaSuccess && coop && opt(kernel, R::kSmem) &&
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kResThreads, R::kSmem) == cudaSuccess && per_sm >= 1) {
            c.ctas = sm_count();   // one CTA per SM: it uses all of the SM's shared memory
            c.checked = 1;
        } else {
            cudaGetLastError();
            c.checked = -1;
        }
    }
    if (c.checked < 0 || nt64 > (int64_t)c.ctas * R::kSlots) return kErrUnsupportedShape;
    CUtensorMap map;
    if (!make_whole_tile_map(&map, a.in, a.rows, a.cols, T::kBytesPerElem)) return kErrUnsupportedShape;
    int rc = launch_zero_scalars(a.ws, st);
    if (rc) return rc;
    int n_tiles = (int)nt64, blocks_x = (int)bx, ss = a.ss_mode, nnz_is_i64 = nnz64;
    const int grid = n_tiles < c.ctas ? n_tiles : c.ctas;   // CTA b takes tiles b, b + grid, ...
    void* out = a.out;
    int64_t cols = a.cols;
    float thr = a.threshold;
    float* block_err = a.block_err;
    ScalarsWs* ws = a.ws;
    uint32_t limit = kSpinLimit;
    void* args[] = {&map, &out, &cols, &blocks_x, &n_tiles, &ss, &thr, &block_err, &ws, &meta, &gamax, &gnnz,
                    &nnz_is_i64, &gerr, &limit};
    if (cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3((unsigned)grid), dim3(kResThreads), args,
                                    (size_t)R::kSmem, st) != cudaSuccess) {
        cudaGetLastError();
        return kErrLaunch;
    }
    return kOk;
}

}  // namespace

// kErrUnsupportedShape: the tensor is not one this kernel takes (too large, other blocks, a device
// without cooperative launch) and the caller runs the sequence of launches instead.
int launch_block_resident(const ScalingArgs& a, int32_t* meta, float* gamax, void* gnnz, int nnz_is_i64, float* gerr,
                          cudaStream_t st) {
    if (a.brows != 128 || a.bcols != 128 || resident_disabled() || force_generic()) return kErrUnsupportedShape;
    if (a.rows % 128 || a.cols % 128 || a.rows >= (int64_t(1) << 31) || a.cols >= (int64_t(1) << 31)) return kErrUnsupportedShape;
    const bool e8 = a.ss_mode == 2;
    if (a.is_fp32) return e8 ? launch_resident_t<Fp32, true>(a, meta, gamax, gnnz, nnz_is_i64, gerr, st)
                             : launch_resident_t<Fp32, false>(a, meta, gamax, gnnz, nnz_is_i64, gerr, st);
    return e8 ? launch_resident_t<Bf16, true>(a, meta, gamax, gnnz, nnz_is_i64, gerr, st)
              : launch_resident_t<Bf16, false>(a, meta, gamax, gnnz, nnz_is_i64, gerr, st);
}

}  // namespace morb
