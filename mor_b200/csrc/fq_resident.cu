// fake_quantize_block_scaling on 128 x 128 blocks as ONE kernel, for tensors small enough to
// stay in the shared memories of the GPU between the two passes (ref: the five launches at
// fake_quantize.cu:2093-2099; the reference authors' cooperative prototype is
// jatin/fake_quantize_num_blocks.cu:973-1233).
//
// One CTA per SM, launched cooperatively so that every CTA is resident.  A CTA owns up to
// kSlots tiles (7 of bf16, 3 of binary32), each handled from start to end by its own group of
// threads (128 for bf16, 256 for binary32), and requests all of them by TMA as it starts: the
// tensor is read from HBM exactly once.
//
//   pass 1   per tile, as it arrives: amax, non-zero count and the screening flags of the short
//            quotient, from shared memory; one atomicMax / atomicAdd per CTA for the tensor.
//   barrier  every CTA now knows the tensor's amax.
//   pass 2   per tile: scale (ref: 1059-1093), E4M3 cast through a table of quotients, store,
//            error sum in the reference's order (ref: 1117-1156).  A thread stands for the
//            logical threads (tx .. tx + VW - 1, ty) and (same, ty + 16) of the reference's
//            32 x 32 CTA: rows ty + 32 j outer, words tx + 32 i inner, high half first, then
//            the reference's two shuffle trees (logical_warp_sum, warp_sum_ordered).
//   barrier  every CTA now sees every block's error sum.
//   decide   every CTA repeats the reference's ordered sum (thread t adds entries t, t + 1024;
//            ref: 1183-1196) -- same additions, same bits -- and, if the tensor stays BF16
//            (ref: 1203-1241), writes its tiles back from shared memory.  The input is never
//            read again, so output == input needs no special order.
//
// Tables.  Under the tensor-wide scale (ss_mode 4) all tiles share one table of RN(q / scale).
// Under the global-mantissa rule (ss_mode 1) every block's scale is the significand of
// 448 / global_amax times a power of two, so all tiles share one table for that significand and
// multiply by their own power of two (PathLutExp); a tile whose exponent would take a quotient
// out of the normal range divides per element instead.  ss_mode 2 (power-of-two scales) needs no
// table.  ss_mode 3 (a different significand per block) is not taken by this kernel.
//
// The two grid barriers are counters in the workspace head (zeroed by the launch before this
// one); every wait -- barrier or TMA -- is bounded, and a wait that runs out is reported as
// meta = -1 instead of hanging the GPU.
#include <type_traits>

#include "kernels.cuh"
#include "e8mx_math.cuh"
#include "scaling_math.cuh"
#include "tma.cuh"

namespace morb {

namespace {

// development hook: a probe that includes this file may define it to record where the time goes
#ifndef MORB_TRACE_POINT
#define MORB_TRACE_POINT(i)
#endif

template <typename T> struct Res {
    static constexpr int kTileBytes = 128 * 128 * T::kBytesPerElem;
    static constexpr int kSlots = T::kBytesPerElem == 2 ? 7 : 3;         // tiles (= thread groups) per CTA
    static constexpr int kGroupThreads = T::kBytesPerElem == 2 ? 128 : 256;
    static constexpr int kThreads = kSlots * kGroupThreads;               // 896 / 768
    static constexpr int kVecPerRow = 128 * T::kBytesPerElem / 16;        // 16 / 32
    static constexpr int kLanesPerRow = kVecPerRow / 2;                   // a lane takes vectors p and p + kLanesPerRow
    // behind the tiles: mbarriers, per-tile statistics and scales, warp sums, one quotient table
    static constexpr int kBarOff = kSlots * kTileBytes;   // 8 x uint64
    static constexpr int kAmaxOff = kBarOff + 64;          // 8 x uint32  tile amax bits
    static constexpr int kNnzOff = kAmaxOff + 32;          // 8 x int32   tile non-zero count
    static constexpr int kFlagOff = kNnzOff + 32;          // 8 x uint32  bit 0: short quotient not allowed, bit 1: NaN seen
    static constexpr int kSfOff = kFlagOff + 32;           // 8 x float   tile scale
    static constexpr int kMiscOff = kSfOff + 32;           // 8 x uint32
    static constexpr int kWsumOff = kMiscOff + 32;         // kSlots x 32 x float (also the 32 partial sums of the decision)
    static constexpr int kLutOff = kWsumOff + kSlots * 128;
    static constexpr int kSmem = kLutOff + 1024;
    static_assert(kLutOff % 16 == 0, "table alignment");
    static_assert(kSmem <= 227 * 1024, "shared memory of one SM");
};

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// barrier among the `count` threads (a multiple of 32) that name the same id (1 .. 15)
__device__ __forceinline__ void group_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// All CTAs of the (cooperative) grid meet here.  False for every thread of the CTA if the
// others did not show up within the limit.
__device__ __forceinline__ bool grid_barrier(uint32_t* counter, uint32_t expected, uint32_t limit) {
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) {
        uint32_t seen;
        // release: what this CTA wrote before is visible to whoever sees the count; acquire: and the reverse
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(seen) : "l"(counter) : "memory");
        uint32_t polls = 0;
        if (seen + 1u < expected) {   // the last one to arrive does not have to look again
            while (ld_acquire_gpu(counter) < expected) {
                if (++polls > limit) { ok = false; break; }
            }
        }
    }
    return __syncthreads_and(ok) != 0;
}

// pass 2 of one tile by its thread group; returns the error sums of the two logical warps (rows ty
// and ty + 16) this lane belongs to, valid in the lanes with p == 0
template <typename T, int DIV, bool NOZERO, typename P>
__device__ __forceinline__ void cast_tile(const P& path, const typename T::vec_t* tile, typename T::vec_t* dst,
                                          int64_t cols_vec, int p, int tyh, float& sum0, float& sum1) {
    using R = Res<T>;
    constexpr int VW = T::kWordsPerVec, VPR = R::kVecPerRow, LPR = R::kLanesPerRow;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int ty = tyh + 16 * half;
        const typename T::vec_t* src = tile + ty * VPR + p;
        typename T::vec_t* o = dst + (int64_t)ty * cols_vec + p;
        float acc[VW];
#pragma unroll
        for (int k = 0; k < VW; ++k) acc[k] = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                typename T::vec_t out;
                err_vec<T, P, true, DIV, NOZERO>(path, src[j * 32 * VPR + i * LPR], out, acc);
                st_stream(o + i * LPR, out);
            }
            o += 32 * cols_vec;
        }
        const float s = logical_warp_sum<VW>(acc);
        if (half == 0) sum0 = s; else sum1 = s;
    }
}

template <typename T, bool E8>
__global__ void __launch_bounds__(Res<T>::kThreads, 1)
block_resident_kernel(const __grid_constant__ CUtensorMap tmap, void* __restrict__ out_raw, int64_t cols, int blocks_x,
                      int n_tiles, int ss, float threshold, float* __restrict__ block_err, ScalarsWs* __restrict__ ws,
                      int32_t* __restrict__ meta_out, float* __restrict__ gamax_out, void* __restrict__ gnnz_out,
                      int nnz_is_i64, float* __restrict__ gerr_out, uint32_t spin_limit) {
    using R = Res<T>;
    using V = typename T::vec_t;
    constexpr int GT = R::kGroupThreads, NT = R::kThreads;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + R::kBarOff);
    uint32_t* s_amax = reinterpret_cast<uint32_t*>(smem + R::kAmaxOff);
    int* s_nnz = reinterpret_cast<int*>(smem + R::kNnzOff);
    uint32_t* s_flag = reinterpret_cast<uint32_t*>(smem + R::kFlagOff);
    float* s_sf = reinterpret_cast<float*>(smem + R::kSfOff);
    uint32_t* s_misc = reinterpret_cast<uint32_t*>(smem + R::kMiscOff);
    float* s_wsum = reinterpret_cast<float*>(smem + R::kWsumOff);
    float* s_lut = reinterpret_cast<float*>(smem + R::kLutOff);

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = tid / GT, gt = tid % GT;            // thread group = tile slot, thread within the group
    const int G = gridDim.x;
    // this CTA's tiles: blockIdx.x, blockIdx.x + G, ...
    const int n_mine = (n_tiles - (int)blockIdx.x + G - 1) / G;   // 1 .. kSlots (the launcher guarantees it)
    const bool have = g < n_mine;
    const int t = (int)blockIdx.x + g * G;             // this group's tile
    const int bx = have ? t % blocks_x : 0, by = have ? t / blocks_x : 0;
    const V* tile = reinterpret_cast<const V*>(smem + g * R::kTileBytes);

    if (tid == 0) MORB_TRACE_POINT(0);
    if (tid == 0) {
        for (int k = 0; k < R::kSlots; ++k) mbar_init(&s_bar[k], 1);
    }
    if (tid < 8) { s_amax[tid] = 0u; s_nnz[tid] = 0; s_flag[tid] = 0u; }
    __syncthreads();
    if (gt == 0 && have) {
        mbar_expect_tx(&s_bar[g], R::kTileBytes);
        tma_load_2d(smem + g * R::kTileBytes, &tmap, bx * 128, by * 128, &s_bar[g]);
    }

    // ---- pass 1: statistics of the group's tile, as soon as it has arrived ---------------
    bool arrived = true;
    if (have) {
        arrived = __all_sync(0xFFFFFFFFu, mbar_wait_bounded(&s_bar[g], 0));   // warp-uniform
        if (gt == 0) MORB_TRACE_POINT(8 + g);
        if (arrived) {
            constexpr int kVecPerThread = R::kTileBytes / 16 / GT;   // 16
            uint32_t amax_bits, flags = 0u;
            int nnz = 0;
            if constexpr (T::kBytesPerElem == 2) {
                uint32_t pmx = 0u, pmn = 0x7FFF7FFFu;
                int nnz4 = 0;
#pragma unroll 4
                for (int u = 0; u < kVecPerThread; ++u) {
                    const uint4 v = tile[gt + u * GT];
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
                float a = 0.0f;
#pragma unroll 4
                for (int u = 0; u < kVecPerThread; ++u) {
                    const float4 v = tile[gt + u * GT];
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
                atomicMax(&s_amax[g], amax_bits);
                if (nnz) atomicAdd(&s_nnz[g], nnz);
                if (flags) atomicOr(&s_flag[g], flags);
            }
        }
    }
    arrived = __syncthreads_and(arrived) != 0;
    if constexpr (T::kBytesPerElem == 2) {
        // a NaN in the tile: the packed maximum is not the reference's (fmaxf ignores NaNs and they are
        // not counted); redo the tile with float compares
        if (have && arrived && (s_flag[g] & 2u)) {   // uniform within the group
            group_sync(1 + g, GT);
            if (gt == 0) { s_amax[g] = 0u; s_nnz[g] = 0; }
            group_sync(1 + g, GT);
            float a = 0.0f;
            int n = 0;
            for (int u = 0; u < R::kTileBytes / 16 / GT; ++u) {
                const uint4 v = tile[gt + u * GT];
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
            if (lane == 0) { atomicMax(&s_amax[g], f2u(a)); if (n) atomicAdd(&s_nnz[g], n); }
        }
        __syncthreads();
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
    if (tid == 0) MORB_TRACE_POINT(1);
    bool alive = grid_barrier(&ws->bar[0], (uint32_t)G, spin_limit);
    if (tid == 0) MORB_TRACE_POINT(2);
    // a CTA whose tile did not arrive told the others before the barrier: everybody stops here
    alive = alive && *reinterpret_cast<volatile uint32_t*>(&ws->load_timeout) == 0u;
    if (!alive) {
        if (tid == 0) {
            atomicOr(&ws->load_timeout, 1u);
            if (blockIdx.x == 0 && meta_out) *meta_out = -1;
        }
        // give a copy that may still be in flight a last bounded chance before the shared memory is released
        if (have) mbar_wait_bounded(&s_bar[g], 0);
        return;
    }

    // ---- pass 2: scale, cast, store, error sums ---------------------------------------
    const float gamax = u2f(*reinterpret_cast<volatile uint32_t*>(&ws->gamax_bits));
    if (tid < n_mine) s_sf[tid] = scaling_factor(ss, gamax, u2f(s_amax[tid]));
    if constexpr (!E8) {
        // one table for the whole CTA: the tensor-wide scale (ss_mode 4), or the significand that all
        // block scales share under the global-mantissa rule (ss_mode 1)
        if (tid >= NT - 256) {
            float base = scaling_factor(ss, gamax, gamax);
            if (ss == 1) base = u2f(0x3F800000u | (f2u(base) & 0x007FFFFFu));
            fill_lut32(s_lut, base, tid - (NT - 256), 256);
        }
    }
    __syncthreads();
    if (have) {
        const int p = gt % R::kLanesPerRow, tyh = gt / R::kLanesPerRow;   // tyh: 0 .. 15
        const int64_t cols_vec = cols * T::kBytesPerElem / 16;
        V* dst = static_cast<V*>(out_raw) + (int64_t)by * 128 * cols_vec + (int64_t)bx * R::kVecPerRow;
        const bool zero_free = s_nnz[g] == 128 * 128 && !(s_flag[g] & 2u);
        const bool short_ok = T::kBytesPerElem != 2 || !(s_flag[g] & 1u);
        const float sf = s_sf[g];
        float sum0 = 0.0f, sum1 = 0.0f;
        auto dispatch = [&](const auto& path) {
            using P = std::decay_t<decltype(path)>;
            constexpr int kShort = T::kBytesPerElem == 2 ? kDivBf16 : kDivIeee;
            constexpr int kLong = T::kBytesPerElem == 2 ? kDivBf16Any : kDivIeee;
            if (short_ok && zero_free) cast_tile<T, kShort, true, P>(path, tile, dst, cols_vec, p, tyh, sum0, sum1);
            else if (short_ok) cast_tile<T, kShort, false, P>(path, tile, dst, cols_vec, p, tyh, sum0, sum1);
            else cast_tile<T, kLong, false, P>(path, tile, dst, cols_vec, p, tyh, sum0, sum1);
        };
        if constexpr (E8) {
            dispatch(PathE8{e8_consts(sf)});
        } else {
            const uint32_t field = (f2u(sf) >> 23) & 0xFFu;
            if (ss != 1) dispatch(PathLut{s_lut, sf});
            else if (field >= 12u && field <= 240u) dispatch(PathLutExp{s_lut, sf, u2f((254u - field) << 23)});
            else dispatch(PathDiv{sf});
        }
        float* wsum = s_wsum + g * 32;
        if (p == 0) { wsum[tyh] = sum0; wsum[tyh + 16] = sum1; }
        group_sync(1 + g, GT);
        if (gt < 32) {
            const float tot = warp_sum_ordered(wsum[gt]);
            if (gt == 0) block_err[t] = tot;
        }
    }
    if (tid == 0) MORB_TRACE_POINT(3);
    const bool met = grid_barrier(&ws->bar[1], (uint32_t)G, spin_limit);
    if (tid == 0) MORB_TRACE_POINT(4);
    if (!met) {
        if (tid == 0) {
            atomicOr(&ws->load_timeout, 1u);
            if (blockIdx.x == 0 && meta_out) *meta_out = -1;
        }
        return;
    }

    // ---- decision: every CTA repeats the ordered sum of all blocks' errors -------------
    // logical thread l of 1024 adds entries l, l + 1024, ...; logical warp w = threads 32 w .. 32 w + 31
    for (int w = wid; w < 32; w += NT / 32) {
        float acc = 0.0f;
        for (int e = w * 32 + lane; e < n_tiles; e += 1024) acc = __fadd_rn(acc, __ldcg(block_err + e));
        acc = warp_sum_ordered(acc);
        if (lane == 0) s_wsum[w] = acc;
    }
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
    if (tid == 0) MORB_TRACE_POINT(5);
    if (s_misc[0] && have) {
        // the tensor stays as it was: the tile is still in shared memory
        constexpr int VPR = R::kVecPerRow;
        const int64_t cols_vec = cols * T::kBytesPerElem / 16;
        V* out_v = static_cast<V*>(out_raw) + (int64_t)by * 128 * cols_vec + (int64_t)bx * VPR;
        for (int v = gt; v < 128 * VPR; v += GT) st_stream(out_v + (int64_t)(v / VPR) * cols_vec + (v % VPR), tile[v]);
    }
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
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, R::kThreads, R::kSmem) == cudaSuccess && per_sm >= 1) {
            c.ctas = sm_count();   // one CTA per SM: it uses all of the SM's shared memory
            c.checked = 1;
        } else {
            cudaGetLastError();
            c.checked = -1;
        }
    }
    if (c.checked < 0 || nt64 > (int64_t)c.ctas * R::kSlots) return kErrUnsupportedShape;
    CUtensorMap map;
    // one box = one whole 128 x 128 tile, row-major in shared memory
    if (!make_tile_map(&map, a.in, a.rows, a.cols, T::kBytesPerElem, 128, 128)) return kErrUnsupportedShape;
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
    if (cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3((unsigned)grid), dim3(R::kThreads), args,
                                    (size_t)R::kSmem, st) != cudaSuccess) {
        // e.g. fewer SMs than the device reports are available to this process: the grid cannot be resident.
        // Nothing has run yet (the scalars were zeroed, which the launch sequence does again): take that one,
        // now and from here on.
        cudaGetLastError();
        c.checked = -1;
        return kErrUnsupportedShape;
    }
    return kOk;
}

// ---------------------------------------------------------------------------------
// quantize_e8mx in one launch (ref: 1361-1428: amax kernel, then the element kernel)
// ---------------------------------------------------------------------------------
// The same idea on a flat tensor: CTA b requests chunks b, b + grid, ... (32 KiB each, up to seven) with bulk
// copies as it starts, takes the largest magnitude from shared memory as they land (NaNs skipped, as the
// reference's fmaxf does), meets the other CTAs at one grid barrier, and casts from shared memory with the
// tensor's scale.  HBM is read once.  A chunk whose copy does not land within the bounded wait is read with
// ordinary loads instead.
constexpr int kE8Chunk = 32 * 1024, kE8Slots = 7, kE8Threads = 1024;
constexpr int kE8Smem = kE8Slots * kE8Chunk + 64 + 512;   // chunks, mbarriers, the 128 offsets of the cast

template <int M>
__global__ void __launch_bounds__(kE8Threads, 1)
e8mx_resident_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int64_t n_bytes, int strategy,
                     ScalarsWs* __restrict__ ws, uint32_t limit) {
    extern __shared__ __align__(128) uint8_t s_data[];
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_data + kE8Slots * kE8Chunk);
    uint32_t* s_off = reinterpret_cast<uint32_t*>(s_data + kE8Slots * kE8Chunk + 64);
    __shared__ uint32_t s_red[kE8Threads / 32];
    const int tid = threadIdx.x;
    const int64_t n_chunks = (n_bytes + kE8Chunk - 1) / kE8Chunk;
    auto chunk_of = [&](int k) { return (int64_t)blockIdx.x + (int64_t)k * gridDim.x; };
    auto bytes_of = [&](int64_t c) { const int64_t r = n_bytes - c * kE8Chunk; return (uint32_t)(r < kE8Chunk ? r : kE8Chunk); };
    if (tid == 0) {
#pragma unroll
        for (int k = 0; k < kE8Slots; ++k) mbar_init(&s_bar[k], 1);
    }
    __syncthreads();
    if (tid == 0) {
        for (int k = 0; k < kE8Slots; ++k) {
            const int64_t c = chunk_of(k);
            if (c >= n_chunks) break;
            mbar_expect_tx(&s_bar[k], bytes_of(c));
            bulk_load(s_data + k * kE8Chunk, in + c * kE8Chunk, bytes_of(c), &s_bar[k]);
        }
    }
    // pass 1: the largest magnitude, two halves of a word at a time; a NaN pattern sorts above infinity and is dropped
    uint32_t pmx = 0u;
    bool all_landed = true;
    for (int k = 0; k < kE8Slots; ++k) {
        const int64_t c = chunk_of(k);
        if (c >= n_chunks) break;
        const bool landed = mbar_wait_bounded(&s_bar[k], 0);
        all_landed = all_landed && landed;
        uint4* v = reinterpret_cast<uint4*>(s_data + k * kE8Chunk);
        const uint4* g = reinterpret_cast<const uint4*>(in + c * kE8Chunk);
        const int nv = (int)(bytes_of(c) / 16);
        for (int i = tid; i < nv; i += kE8Threads) {
            uint4 x;
            if (landed) x = v[i];
            else { x = ld_stream(g + i); v[i] = x; }   // this thread reads the same vectors again in pass 2
            uint32_t m[4] = {mag2(x.x), mag2(x.y), mag2(x.z), mag2(x.w)};
            uint32_t mx = umax16x2_3(umax16x2_3(m[0], m[0], m[1]), m[2], m[3]);
            if (umin16x2(mx, 0x7F807F80u) != mx) {
                mx = 0u;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t lo = m[q] & 0xFFFFu, hi = m[q] >> 16;
                    lo = lo > 0x7F80u ? 0u : lo;
                    hi = hi > 0x7F80u ? 0u : hi;
                    mx = umax16x2(mx, lo | (hi << 16));
                }
            }
            pmx = umax16x2(pmx, mx);
        }
    }
    const uint32_t top = __reduce_max_sync(0xFFFFFFFFu, hmax_halves(pmx));
    if ((tid & 31) == 0) s_red[tid >> 5] = top;
    __syncthreads();
    if (tid == 0) {
        uint32_t a = 0u;
#pragma unroll
        for (int w = 0; w < kE8Threads / 32; ++w) a = max(a, s_red[w]);
        atomicMax(&ws->gamax_bits, a << 16);
    }
    const bool met = grid_barrier(&ws->bar[0], gridDim.x, limit);
    if (met) {
        // pass 2: the cast, from shared memory
        E8mxCast<M> cast;
        cast.init(s_off, e8mx_scale<M>(u2f(ld_acquire_gpu(&ws->gamax_bits)), strategy), tid);
        __syncthreads();
        for (int k = 0; k < kE8Slots; ++k) {
            const int64_t c = chunk_of(k);
            if (c >= n_chunks) break;
            const uint4* v = reinterpret_cast<const uint4*>(s_data + k * kE8Chunk);
            uint4* o = reinterpret_cast<uint4*>(out + c * kE8Chunk);
            const int nv = (int)(bytes_of(c) / 16);
            for (int i = tid; i < nv; i += kE8Threads) {
                const uint4 x = v[i];
                uint4 r;
                r.x = cast.word(x.x); r.y = cast.word(x.y); r.z = cast.word(x.z); r.w = cast.word(x.w);
                st_stream(o + i, r);
            }
        }
    } else if (tid == 0) {
        atomicOr(&ws->load_timeout, 1u);   // the other CTAs did not show up: nothing is written
    }
    if (!all_landed) {
        // a copy may still be in flight: one more bounded chance to land before the shared memory is handed on
        for (int k = 0; k < kE8Slots; ++k)
            if (chunk_of(k) < n_chunks) mbar_wait_bounded(&s_bar[k], 0);
    }
}

template <int M>
int launch_e8mx_resident_t(const void* in, void* out, int64_t n_bytes, int strategy, ScalarsWs* ws, cudaStream_t st) {
    static DeviceCaps caps[64];
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kErrUnsupportedShape;
    DeviceCaps& c = caps[dev];
    auto kernel = e8mx_resident_kernel<M>;
    if (c.checked == 0) {
        int coop = 0, per_sm = 0;
        static SmemOptIn opt;
        if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) == cudaSuccess && coop && opt(kernel, kE8Smem) &&
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kE8Threads, kE8Smem) == cudaSuccess && per_sm >= 1) {
            c.ctas = sm_count();
            c.checked = 1;
        } else {
            cudaGetLastError();
            c.checked = -1;
        }
    }
    const int64_t n_chunks = (n_bytes + kE8Chunk - 1) / kE8Chunk;
    if (c.checked < 0 || n_chunks > (int64_t)c.ctas * kE8Slots) return kErrUnsupportedShape;
    const int rc = launch_zero_scalars(ws, st);
    if (rc) return rc;
    const int grid = (int)(n_chunks < c.ctas ? n_chunks : c.ctas);
    const uint8_t* in8 = static_cast<const uint8_t*>(in);
    uint8_t* out8 = static_cast<uint8_t*>(out);
    uint32_t limit = kSpinLimit;
    void* args[] = {&in8, &out8, &n_bytes, &strategy, &ws, &limit};
    if (cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3((unsigned)grid), dim3(kE8Threads), args,
                                    (size_t)kE8Smem, st) != cudaSuccess) {
        cudaGetLastError();   // the grid cannot be resident: the launch sequence takes over, now and from here on
        c.checked = -1;
        return kErrUnsupportedShape;
    }
    return kOk;
}

}  // namespace

// kErrUnsupportedShape: the tensor is not one this kernel takes (too large, other blocks, ss_mode 3, a
// device without cooperative launch) and the caller runs the sequence of launches instead.
int launch_block_resident(const ScalingArgs& a, int32_t* meta, float* gamax, void* gnnz, int nnz_is_i64, float* gerr,
                          cudaStream_t st) {
    if (a.brows != 128 || a.bcols != 128 || a.ss_mode == 3 || resident_disabled() || force_generic()) return kErrUnsupportedShape;
    if (a.rows % 128 || a.cols % 128 || a.rows >= (int64_t(1) << 31) || a.cols >= (int64_t(1) << 31)) return kErrUnsupportedShape;
    const bool e8 = a.ss_mode == 2;
    if (a.is_fp32) return e8 ? launch_resident_t<Fp32, true>(a, meta, gamax, gnnz, nnz_is_i64, gerr, st)
                             : launch_resident_t<Fp32, false>(a, meta, gamax, gnnz, nnz_is_i64, gerr, st);
    return e8 ? launch_resident_t<Bf16, true>(a, meta, gamax, gnnz, nnz_is_i64, gerr, st)
              : launch_resident_t<Bf16, false>(a, meta, gamax, gnnz, nnz_is_i64, gerr, st);
}

// kErrUnsupportedShape: not a tensor for the single launch (too large, a length that is no multiple of 16 bytes,
// no cooperative launch): the caller runs the amax kernel and the element kernel instead.
int launch_e8mx_resident(const void* in, void* out, int64_t n_elems, int qtype, int strategy, ScalarsWs* ws,
                         cudaStream_t st) {
    const int64_t n_bytes = n_elems * 2;
    if (n_bytes % 16 || resident_disabled() || force_generic()) return kErrUnsupportedShape;
    switch (qtype) {
        case 1: return launch_e8mx_resident_t<1>(in, out, n_bytes, strategy, ws, st);
        case 2: return launch_e8mx_resident_t<2>(in, out, n_bytes, strategy, ws, st);
        case 3: return launch_e8mx_resident_t<3>(in, out, n_bytes, strategy, ws, st);
        default: return kErrInvalidArgument;
    }
}

}  // namespace morb
