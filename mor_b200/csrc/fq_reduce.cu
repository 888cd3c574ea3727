// amax / non-zero reductions (ref: 951-1049, 1459-1631).  max and integer sums are
// order-independent, so these kernels are free to use any traversal: 16-byte loads,
// warp shuffles, one shared-memory step per CTA, and one atomicMax / atomicAdd per CTA
// into the workspace scalars (the bit pattern of a non-negative float orders like an
// unsigned integer).
//
// These kernels read 2 bytes per bf16 element, i.e. they have about 11 issue slots per
// element at the HBM roofline, so bf16 data is reduced in packed form: a magnitude
// word (w & 0x7FFF7FFF) feeds one packed 16-bit maximum for both halves, and the
// non-zero count comes from bit 15 of each half of m + 0x7FFF7FFF.  NaNs, which the
// reference's fmaxf ignores and never counts, show up as a packed maximum above
// 0x7F80; a CTA that sees one redoes its part with float compares.
#include "kernels.cuh"
#include "p2p.cuh"
#include "tma.cuh"

namespace morb {

namespace {

constexpr int kThreads = 256;

struct Acc {
    uint32_t packed_max;  // bf16 path: two 15-bit maxima
    float fmax_;          // float path
    int nnz;              // bf16 path: four times the count
    uint32_t tmin;        // bf16 path: packed signed minimum of (magnitude + 0x7FFF) per half, starts at 0x7FFF7FFF
};
__device__ __forceinline__ Acc acc_init() { return Acc{0u, 0.0f, 0, 0x7FFF7FFFu}; }

// true when a half of the packed minimum stands for a non-zero magnitude below 2^-90
// (bf16 pattern 0x1280): a zero leaves 0x7FFF, a magnitude m leaves 0x8000 + m - 1
__device__ __forceinline__ bool tmin_is_tiny(uint32_t t) {
    return (t & 0x7FFFu) < 0x127Fu || ((t >> 16) & 0x7FFFu) < 0x127Fu;
}

template <typename T>
__device__ __forceinline__ void vec_acc_fast(const typename T::vec_t& v, Acc& a) {
    if constexpr (T::kBytesPerElem == 2) {
        // s = m + 0x7FFF per half: bit 15 says "non-zero", and as a signed 16-bit number s
        // orders the non-zero magnitudes below every zero, so one packed minimum tracks the
        // smallest non-zero magnitude; the eight "non-zero" bits are spread to nibbles and
        // counted by one popcount
        const uint32_t m0 = mag2(v.x), m1 = mag2(v.y), m2 = mag2(v.z), m3 = mag2(v.w);
        a.packed_max = umax16x2_3(umax16x2_3(a.packed_max, m0, m1), m2, m3);
        const uint32_t s0 = m0 + 0x7FFF7FFFu, s1 = m1 + 0x7FFF7FFFu, s2 = m2 + 0x7FFF7FFFu, s3 = m3 + 0x7FFF7FFFu;
        a.tmin = smin16x2_3(smin16x2_3(a.tmin, s0, s1), s2, s3);
        const uint32_t p01 = top_bits_to_bytes(s0, s1), p23 = top_bits_to_bytes(s2, s3);
        a.nnz += __popc((p01 & 0x0F0F0F0Fu) | (p23 & 0xF0F0F0F0u));
    } else {
        const float a0 = fabsf(v.x), a1 = fabsf(v.y), a2 = fabsf(v.z), a3 = fabsf(v.w);
        a.fmax_ = fmaxf(fmaxf(a.fmax_, a0), fmaxf(fmaxf(a1, a2), a3));
        a.nnz += (a0 > 0.0f) + (a1 > 0.0f) + (a2 > 0.0f) + (a3 > 0.0f);
    }
}
template <typename T>
__device__ __forceinline__ int acc_nnz(const Acc& a) {
    if constexpr (T::kBytesPerElem == 2) return a.nnz >> 2;
    else return a.nnz;
}
template <typename T>
__device__ __forceinline__ bool acc_tiny(const Acc& a) {
    if constexpr (T::kBytesPerElem == 2) return tmin_is_tiny(a.tmin);
    else return false;
}
template <typename T>
__device__ __forceinline__ void vec_acc_exact(const typename T::vec_t& v, float& amax, int& nnz) {
#pragma unroll
    for (int k = 0; k < T::kWordsPerVec; ++k) {
        float hi, lo;
        T::unpack(v, k, hi, lo);
        const float ah = fabsf(hi), al = fabsf(lo);
        amax = fmaxf(amax, fmaxf(ah, al));
        nnz += (ah > 0.0f) + (al > 0.0f);
    }
}

// CTA-wide combine; totals valid in thread 0 (and in all of warp 0's lanes).
__device__ __forceinline__ void cta_combine(float& amax, int& nnz) {
    __shared__ float s_a[32];
    __shared__ int s_n[32];
    __syncthreads();
    amax = warp_max(amax);
    nnz = warp_sum_int(nnz);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { s_a[wid] = amax; s_n[wid] = nnz; }
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    amax = lane < nw ? s_a[lane] : 0.0f;
    nnz = lane < nw ? s_n[lane] : 0;
    amax = warp_max(amax);
    nnz = warp_sum_int(nnz);
}

// One-barrier CTA reduction of (amax bits, count, flag bits); every thread gets the totals.
// amax must be non-negative (or a NaN pattern, which then wins the unsigned maximum).
__device__ __forceinline__ void cta_reduce_all(float& amax, int& nnz, uint32_t& flags) {
    __shared__ uint32_t s_a[32], s_f[32];
    __shared__ int s_n[32];
    uint32_t ab = __reduce_max_sync(0xFFFFFFFFu, f2u(amax));
    nnz = __reduce_add_sync(0xFFFFFFFFu, nnz);
    flags = __reduce_or_sync(0xFFFFFFFFu, flags);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { s_a[wid] = ab; s_n[wid] = nnz; s_f[wid] = flags; }
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    ab = __reduce_max_sync(0xFFFFFFFFu, lane < nw ? s_a[lane] : 0u);
    nnz = __reduce_add_sync(0xFFFFFFFFu, lane < nw ? s_n[lane] : 0);
    flags = __reduce_or_sync(0xFFFFFFFFu, lane < nw ? s_f[lane] : 0u);
    amax = u2f(ab);
}
constexpr uint32_t kFlagTiny = 1u, kFlagNan = 2u;
template <typename T>
__device__ __forceinline__ uint32_t acc_flags(const Acc& a, float amax) {
    if constexpr (T::kBytesPerElem == 2) return (tmin_is_tiny(a.tmin) ? kFlagTiny : 0u) | (f2u(amax) > 0x7F800000u ? kFlagNan : 0u);
    else return 0u;
}

template <typename T>
__device__ __forceinline__ float acc_amax(const Acc& a) {
    if constexpr (T::kBytesPerElem == 2) return u2f(hmax_halves(a.packed_max) << 16);
    else return a.fmax_;
}
__device__ __forceinline__ void publish(ScalarsWs* ws, float amax, int nnz) {
    atomicMax(&ws->gamax_bits, f2u(amax));
    if (nnz) atomicAdd(&ws->gnnz, (unsigned long long)nnz);
}
__global__ void zero_scalars_kernel(ScalarsWs* ws) {
    // the amax kernel behind this one may start reading the tensor now; it waits for this kernel before its first atomic
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    ws->gamax_bits = 0u; ws->fallback = 0; ws->gnnz = 0ull; ws->gerr = 0.0f; ws->meta = 0;
    ws->div_unsafe = 0u; ws->load_timeout = 0u; ws->bar[0] = 0u; ws->bar[1] = 0u;
}

// Flat tensor: every warp streams its own 4 KiB chunks through a private two-stage
// shared-memory ring filled by bulk copies (two chunks per warp, both requested as the
// warp starts; the grid covers the tensor once, so the hardware's CTA scheduler evens
// out the SMs).
constexpr int kFlatStages = 2, kFlatChunkVec = 256, kFlatWarps = kThreads / 32;
template <typename T>
__global__ void __launch_bounds__(kThreads) amax_nnz_flat_kernel(const typename T::vec_t* __restrict__ in,
                                                                 int64_t nvec, int64_t n_tail_elems,
                                                                 ScalarsWs* __restrict__ ws) {
    extern __shared__ __align__(128) uint8_t s_ring[];  // [warp][stage][4 KiB]
    __shared__ __align__(8) uint64_t s_bar[kFlatWarps][kFlatStages];
    using V = typename T::vec_t;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t n_warps = (int64_t)gridDim.x * kFlatWarps, gw = (int64_t)blockIdx.x * kFlatWarps + wid;
    const int64_t gtid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const int64_t n_chunks = (nvec + kFlatChunkVec - 1) / kFlatChunkVec;
    WarpStream<kFlatStages, kFlatChunkVec * 16> stream;
    stream.start(s_ring + wid * (kFlatStages * kFlatChunkVec * 16), s_bar[wid], in, nvec * 16, gw, n_warps);
    Acc acc = acc_init();
    int st = 0;
    for (int64_t c = gw; c < n_chunks; c += n_warps) {
        const int64_t v0 = c * kFlatChunkVec;
        const int nv = (int)(nvec - v0 < kFlatChunkVec ? nvec - v0 : kFlatChunkVec);
        if (stream.acquire(st)) {
            const V* chunk = reinterpret_cast<const V*>(stream.stage(st)) + lane;
#pragma unroll
            for (int r = 0; r < kFlatChunkVec / 32; ++r)
                if (r * 32 + lane < nv) vec_acc_fast<T>(chunk[r * 32], acc);
        } else {
            for (int r = lane; r < nv; r += 32) vec_acc_fast<T>(ld_keep(in + v0 + r), acc);
        }
        stream.release(st, c + kFlatStages * n_warps);
        st = st + 1 == kFlatStages ? 0 : st + 1;
    }
    stream.drain();
    float amax = acc_amax<T>(acc);
    int nnz = acc_nnz<T>(acc);
    uint32_t flags = acc_flags<T>(acc, amax);
    if (gtid < n_tail_elems) {
        float a;
        if constexpr (T::kBytesPerElem == 2) a = fabsf(u2f((uint32_t)reinterpret_cast<const uint16_t*>(in + nvec)[gtid] << 16));
        else a = fabsf(reinterpret_cast<const float*>(in + nvec)[gtid]);
        if (a > 0.0f) {  // false for a NaN, which the maximum has to skip
            amax = fmaxf(amax, a);
            nnz += 1;
            if (a < 8.0779357e-28f) flags |= kFlagTiny;  // 2^-90
        }
    }
    cta_reduce_all(amax, nnz, flags);
    if (flags & kFlagNan) {  // a NaN somewhere in this CTA's part: float compares, as the reference does
        amax = 0.0f; nnz = 0;
        for (int64_t c = gw; c < n_chunks; c += n_warps) {
            const int64_t v0 = c * kFlatChunkVec;
            const int nv = (int)(nvec - v0 < kFlatChunkVec ? nvec - v0 : kFlatChunkVec);
            for (int r = lane; r < nv; r += 32) vec_acc_exact<T>(ld_keep(in + v0 + r), amax, nnz);
        }
        if (gtid < n_tail_elems) {
            float a;
            if constexpr (T::kBytesPerElem == 2) a = fabsf(u2f((uint32_t)reinterpret_cast<const uint16_t*>(in + nvec)[gtid] << 16));
            else a = fabsf(reinterpret_cast<const float*>(in + nvec)[gtid]);
            amax = fmaxf(amax, a);
            nnz += a > 0.0f;
        }
        cta_combine(amax, nnz);
    }
    if (threadIdx.x == 0) {
        publish(ws, amax, nnz);
        if (flags) atomicOr(&ws->div_unsafe, 1u);
    }
}

// The warp that exchanges the slab's scalars with the other ranks from inside the amax kernel: waits (bounded) until
// every CTA of the grid has counted itself in, then publishes and gathers.  Not inlined: its registers are not the
// amax loop's business.
__device__ __noinline__ void last_cta_exchange(ScalarsWs* ws, const PeerFuse* fusep) {
    const PeerFuse& fuse = *fusep;
    bool all_in = false;
    if ((threadIdx.x & 31) == 0) {
        for (uint32_t i = 0; i < kSpinLimit; ++i) {
            uint32_t seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(&ws->bar[0]) : "memory");
            if (seen >= gridDim.x) { all_in = true; break; }
            __nanosleep(100);
        }
        if (!all_in) atomicOr(&ws->load_timeout, 1u);   // reported as meta = -1 by the decision kernel
    }
    all_in = __shfl_sync(0xFFFFFFFFu, (int)all_in, 0) != 0;
    if (all_in)
        exchange_scalars_warp(ws, fuse.mine, fuse.peers, fuse.rank, fuse.world, fuse.epoch, fuse.gamax_out, fuse.gnnz_out,
                              fuse.limit);
}

// One CTA per (brows x bcols) block.  W lanes (a power of two) span a block row in
// 16-byte vectors, 256 / W rows are in flight per step; no division in the loops.
template <typename T>
__global__ void __launch_bounds__(kThreads, 8) amax_nnz_blocks_kernel(const typename T::vec_t* __restrict__ in,
                                                                   int64_t cols_vec, int brows, int bcols_vec,
                                                                   int64_t blocks_x, int w_shift,
                                                                   float* __restrict__ block_amax,
                                                                   ScalarsWs* __restrict__ ws, const __grid_constant__ PeerFuse fuse) {
    // Launched as a programmatic dependent of the kernel that clears the scalars: the loads below may run before
    // that kernel has finished (the tensor was complete before it started), the results are published after
    // griddepcontrol.wait.  The kernel behind this one (the exchange of the amax between ranks, or the cast) may in
    // turn become resident while this kernel's last CTAs run; it waits for this kernel before it reads anything.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int64_t b = blockIdx.x;
    const int64_t r0 = (b / blocks_x) * brows, c0 = (b % blocks_x) * bcols_vec;
    const int W = 1 << w_shift, RPS = kThreads >> w_shift;
    const int tx = threadIdx.x & (W - 1), ty = threadIdx.x >> w_shift;
    const typename T::vec_t* base = in + r0 * cols_vec + c0;
    Acc acc = acc_init();
    if (brows >= 4 * RPS) {  // tall blocks: four rows in flight per lane, eight CTAs per SM
        for (int cv = tx; cv < bcols_vec; cv += W) {
            int r = ty;
            for (; r + 3 * RPS < brows; r += 4 * RPS) {
                typename T::vec_t v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = ld_keep(base + (int64_t)(r + u * RPS) * cols_vec + cv);
#pragma unroll
                for (int u = 0; u < 4; ++u) vec_acc_fast<T>(v[u], acc);
            }
            for (; r < brows; r += RPS) vec_acc_fast<T>(ld_keep(base + (int64_t)r * cols_vec + cv), acc);
        }
    } else {                 // wide blocks (rows of a matrix): four vectors of a row in flight per lane
        for (int r = ty; r < brows; r += RPS) {
            const typename T::vec_t* row = base + (int64_t)r * cols_vec;
            int cv = tx;
            for (; cv + 3 * W < bcols_vec; cv += 4 * W) {
                typename T::vec_t v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = ld_keep(row + cv + u * W);
#pragma unroll
                for (int u = 0; u < 4; ++u) vec_acc_fast<T>(v[u], acc);
            }
            for (; cv < bcols_vec; cv += W) vec_acc_fast<T>(ld_keep(row + cv), acc);
        }
    }
    float amax = acc_amax<T>(acc);
    int nnz = acc_nnz<T>(acc);
    uint32_t flags = acc_flags<T>(acc, amax);
    cta_reduce_all(amax, nnz, flags);
    if (flags & kFlagNan) {
        amax = 0.0f; nnz = 0;
        for (int cv = tx; cv < bcols_vec; cv += W)
            for (int r = ty; r < brows; r += RPS) vec_acc_exact<T>(ld_keep(base + (int64_t)r * cols_vec + cv), amax, nnz);
        cta_combine(amax, nnz);
    }
    if (threadIdx.x == 0) {
        // the sign bit tells the cast kernel that the block holds no zero (and no NaN: those are
        // not counted), so it may leave out the selects that keep zero elements out of the sums
        const bool zero_free = nnz == brows * bcols_vec * (16 / T::kBytesPerElem);
        block_amax[b] = zero_free ? -amax : amax;
        asm volatile("griddepcontrol.wait;" ::: "memory");   // the scalars have been cleared
        publish(ws, amax, nnz);
        if (flags) atomicOr(&ws->div_unsafe, 1u);
    }
    if (fuse.enabled) {
        // Row-sharded tensors: the CTA with the highest index -- scheduled last, so little is left to wait for --
        // exchanges the slab's amax and count with the other ranks over NVLink itself (stores into every peer's
        // buffer, epoch flags, a bounded wait for theirs), so that the collective needs no launch of its own.  Every
        // CTA counts itself in with a release (its results are visible before the count); the exchanging warp waits,
        // bounded, for the full count.  The counter is the first grid-barrier word of the workspace, cleared with the
        // scalars.
        if (threadIdx.x == 0)
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&ws->bar[0]) : "memory");
        if (blockIdx.x == gridDim.x - 1 && threadIdx.x < 32) last_cta_exchange(ws, &fuse);
    }
}

// 1 x k blocks of at least 4 KiB (a multiple of it): in a row-major tensor they are consecutive
// runs of the flat array, so a warp streams one block through its private ring (chunks one
// after the other) and reduces it alone: no CTA barrier until the eight warps of a CTA combine
// their totals for the one atomic update of the tensor-wide scalars.
template <typename T>
__global__ void __launch_bounds__(kThreads) amax_nnz_runs_kernel(const typename T::vec_t* __restrict__ in,
                                                                 int chunks_per_block, int64_t n_blocks,
                                                                 float* __restrict__ block_amax,
                                                                 ScalarsWs* __restrict__ ws) {
    extern __shared__ __align__(128) uint8_t s_ring[];  // [warp][stage][4 KiB]
    __shared__ __align__(8) uint64_t s_bar[kFlatWarps][kFlatStages];
    using V = typename T::vec_t;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t b = (int64_t)blockIdx.x * kFlatWarps + wid;   // this warp's block
    float amax = 0.0f;
    int nnz = 0;
    uint32_t flags = 0u;
    if (b < n_blocks) {
        const int64_t c0 = b * chunks_per_block;
        const V* src = in + c0 * kFlatChunkVec;
        WarpStream<kFlatStages, kFlatChunkVec * 16> stream;
        stream.start(s_ring + wid * (kFlatStages * kFlatChunkVec * 16), s_bar[wid], src,
                     (int64_t)chunks_per_block * kFlatChunkVec * 16, 0, 1);
        Acc acc = acc_init();
        int st = 0;
        for (int c = 0; c < chunks_per_block; ++c) {
            if (stream.acquire(st)) {
                const V* chunk = reinterpret_cast<const V*>(stream.stage(st)) + lane;
#pragma unroll
                for (int r = 0; r < kFlatChunkVec / 32; ++r) vec_acc_fast<T>(chunk[r * 32], acc);
            } else {
                for (int r = lane; r < kFlatChunkVec; r += 32) vec_acc_fast<T>(ld_keep(src + (int64_t)c * kFlatChunkVec + r), acc);
            }
            stream.release(st, c + kFlatStages);
            st = st + 1 == kFlatStages ? 0 : st + 1;
        }
        stream.drain();
        amax = acc_amax<T>(acc);
        nnz = acc_nnz<T>(acc);
        flags = acc_flags<T>(acc, amax);
        amax = u2f(__reduce_max_sync(0xFFFFFFFFu, f2u(amax)));
        nnz = __reduce_add_sync(0xFFFFFFFFu, nnz);
        flags = __reduce_or_sync(0xFFFFFFFFu, flags);
        if (flags & kFlagNan) {  // a NaN in this block: float compares, as the reference does
            amax = 0.0f; nnz = 0;
            for (int64_t r = lane; r < (int64_t)chunks_per_block * kFlatChunkVec; r += 32) vec_acc_exact<T>(ld_keep(src + r), amax, nnz);
            amax = warp_max(amax);
            nnz = warp_sum_int(nnz);
        }
        if (lane == 0) {
            const bool zero_free = nnz == chunks_per_block * kFlatChunkVec * (16 / T::kBytesPerElem);
            block_amax[b] = zero_free ? -amax : amax;
        }
    }
    // totals of the CTA's eight blocks (every lane of a warp holds its block's totals)
    __shared__ uint32_t s_a[kFlatWarps], s_f[kFlatWarps];
    __shared__ int s_n[kFlatWarps];
    if (lane == 0) { s_a[wid] = f2u(amax); s_n[wid] = nnz; s_f[wid] = flags; }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t a = 0u, f = 0u;
        long long n = 0;
#pragma unroll
        for (int w = 0; w < kFlatWarps; ++w) { a = max(a, s_a[w]); n += s_n[w]; f |= s_f[w]; }
        atomicMax(&ws->gamax_bits, a);
        if (n) atomicAdd(&ws->gnnz, (unsigned long long)n);
        if (f) atomicOr(&ws->div_unsafe, 1u);
    }
}

// Column groups (k x 1): a CTA covers 32 consecutive 16-byte column strips (one warp spans them: 512
// contiguous bytes of a row) and a slice of `rows_per_cta` rows of one row block; its eight warps take
// every eighth row, four loads in flight per lane.  The warps' per-column maxima meet in shared memory
// and one atomicMax per column and CTA goes to block_amax.  bf16 data is screened for the short
// quotient of the cast kernels on the way (every non-zero magnitude in [2^-90, 2^90), no NaN).
template <typename T>
__global__ void __launch_bounds__(kThreads) amax_nnz_colgroups_kernel(const typename T::vec_t* __restrict__ in,
                                                                      int64_t cols_vec, int brows, int rows_per_cta,
                                                                      float* __restrict__ block_amax,
                                                                      ScalarsWs* __restrict__ ws) {
    constexpr int EPV = 16 / T::kBytesPerElem;
    __shared__ float s_cmax[8][32][EPV + 1];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t cv = (int64_t)blockIdx.x * 32 + lane;                  // vector column
    const int64_t rb = blockIdx.y;                                       // row block
    const int seg = blockIdx.z;                                          // slice of the k rows
    float cmax[EPV];
#pragma unroll
    for (int e = 0; e < EPV; ++e) cmax[e] = 0.0f;
    int nnz = 0;
    bool unsafe = false;
    if (cv < cols_vec) {
        const int64_t r_begin = rb * brows + (int64_t)seg * rows_per_cta;
        int64_t r_end = r_begin + rows_per_cta;
        if (r_end > (rb + 1) * (int64_t)brows) r_end = (rb + 1) * (int64_t)brows;
        auto take = [&](const typename T::vec_t& v) {
#pragma unroll
            for (int k = 0; k < T::kWordsPerVec; ++k) {
                float hi, lo;
                T::unpack(v, k, hi, lo);
                const float ah = fabsf(hi), al = fabsf(lo);
                cmax[2 * k] = fmaxf(cmax[2 * k], al);          // fmaxf skips NaNs, as the reference's does
                cmax[2 * k + 1] = fmaxf(cmax[2 * k + 1], ah);
                nnz += (ah > 0.0f) + (al > 0.0f);
                // outside the short quotient's range: NaN, or a non-zero magnitude below 2^-90 or at least 2^90
                unsafe = unsafe || !(ah == 0.0f || (ah >= 8.0779357e-28f && ah < 1.2379400e27f)) ||
                         !(al == 0.0f || (al >= 8.0779357e-28f && al < 1.2379400e27f));
            }
        };
        auto scan = [&](auto&& per_vector) {
            int64_t r = r_begin + wid;
            for (; r + 24 < r_end; r += 32) {
                typename T::vec_t v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = ld_keep(in + (r + 8 * u) * cols_vec + cv);
#pragma unroll
                for (int u = 0; u < 4; ++u) per_vector(v[u]);
            }
            for (; r < r_end; r += 8) per_vector(ld_keep(in + r * cols_vec + cv));
        };
        if constexpr (T::kBytesPerElem == 2) {
            // packed form, both columns of a word at once: unsigned 16-bit maxima of the magnitudes per word
            // position, one signed minimum of magnitude + 0x7FFF over everything (a zero becomes 0x7FFF, the
            // largest; bit 15 of a half says "non-zero"), the non-zero count from those bits.  A NaN pattern sorts
            // above infinity, where fmaxf would skip it: a thread that met one repeats its rows element by element.
            uint32_t cm[4] = {0u, 0u, 0u, 0u}, pmn = 0x7FFF7FFFu;
            int n2 = 0;
            scan([&](const uint4& v) {
                const uint32_t m0 = mag2(v.x), m1 = mag2(v.y), m2 = mag2(v.z), m3 = mag2(v.w);
                cm[0] = umax16x2(cm[0], m0); cm[1] = umax16x2(cm[1], m1);
                cm[2] = umax16x2(cm[2], m2); cm[3] = umax16x2(cm[3], m3);
                const uint32_t t0 = m0 + 0x7FFF7FFFu, t1 = m1 + 0x7FFF7FFFu, t2 = m2 + 0x7FFF7FFFu, t3 = m3 + 0x7FFF7FFFu;
                pmn = smin16x2_3(pmn, t0, t1);
                pmn = smin16x2_3(pmn, t2, t3);
                n2 += __popc(((t0 & 0x80008000u) >> 1) | (t1 & 0x80008000u)) + __popc(((t2 & 0x80008000u) >> 1) | (t3 & 0x80008000u));
            });
            const uint32_t mx = hmax_halves(umax16x2(umax16x2_3(cm[0], cm[1], cm[2]), cm[3]));
            if (mx > 0x7F80u) {
                scan(take);
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) { cmax[2 * k] = u2f(cm[k] << 16); cmax[2 * k + 1] = u2f(cm[k] & 0xFFFF0000u); }
                nnz = n2;
                // smallest non-zero magnitude: a half with bit 15 set holds it, less one, in its low 15 bits
                const uint32_t h0 = pmn & 0xFFFFu, h1 = pmn >> 16;
                uint32_t mn = 0x7FFFu;
                if (h0 & 0x8000u) mn = min(mn, (h0 & 0x7FFFu) + 1u);
                if (h1 & 0x8000u) mn = min(mn, (h1 & 0x7FFFu) + 1u);
                unsafe = mx >= 0x6C80u || mn < 0x1280u;   // outside [2^-90, 2^90)
            }
        } else {
            scan(take);
        }
    }
#pragma unroll
    for (int e = 0; e < EPV; ++e) s_cmax[wid][lane][e] = cmax[e];
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < EPV; ++e) amax = fmaxf(amax, cmax[e]);
    __syncthreads();
    for (int t = threadIdx.x; t < 32 * EPV; t += kThreads) {
        const int l = t / EPV, e = t % EPV;
        float m = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) m = fmaxf(m, s_cmax[w][l][e]);
        const int64_t col_vec = (int64_t)blockIdx.x * 32 + l;
        if (col_vec < cols_vec) atomicMax(reinterpret_cast<uint32_t*>(block_amax) + rb * cols_vec * EPV + col_vec * EPV + e, f2u(m));
    }
    const bool any_unsafe = __syncthreads_or(unsafe) != 0;
    cta_combine(amax, nnz);
    if (threadIdx.x == 0) {
        publish(ws, amax, nnz);
        if (any_unsafe || T::kBytesPerElem != 2) atomicOr(&ws->div_unsafe, 1u);
    }
}

__global__ void zero_floats_kernel(float* p, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = 0.0f;
}

}  // namespace

int launch_zero_scalars(ScalarsWs* ws, cudaStream_t st) {
    zero_scalars_kernel<<<1, 1, 0, st>>>(ws);
    return check_launch();
}

int launch_amax_nnz_flat(const void* in, int is_fp32, int64_t n_elems, ScalarsWs* ws, cudaStream_t st) {
    const int epv = is_fp32 ? 4 : 8;
    const int64_t nvec = n_elems / epv, tail = n_elems % epv;
    constexpr int kRing = kFlatWarps * kFlatStages * kFlatChunkVec * 16;
    constexpr int kChunksPerWarp = 2;
    const int64_t n_chunks = (nvec + kFlatChunkVec - 1) / kFlatChunkVec;
    int64_t want = (n_chunks + kFlatWarps * kChunksPerWarp - 1) / (kFlatWarps * kChunksPerWarp);
    if (want > 0x7FFFFFFF) return kErrTooLarge;
    if (want < 1) want = 1;
    static SmemOptIn opt32, opt16;
    if (!(is_fp32 ? opt32(amax_nnz_flat_kernel<Fp32>, kRing) : opt16(amax_nnz_flat_kernel<Bf16>, kRing))) return kErrLaunch;
    if (is_fp32) amax_nnz_flat_kernel<Fp32><<<(int)want, kThreads, kRing, st>>>(static_cast<const float4*>(in), nvec, tail, ws);
    else amax_nnz_flat_kernel<Bf16><<<(int)want, kThreads, kRing, st>>>(static_cast<const uint4*>(in), nvec, tail, ws);
    return check_launch();
}

int launch_amax_nnz_blocks(const void* in, int is_fp32, int64_t rows, int64_t cols, int brows, int bcols,
                           float* block_amax, ScalarsWs* ws, cudaStream_t st, const PeerFuse* fuse) {
    const int epv = is_fp32 ? 4 : 8;
    if (cols % epv) return kErrUnsupportedShape;
    const int64_t cols_vec = cols / epv;
    if (bcols == 1) {
        if (fuse && fuse->enabled) return kErrUnsupportedShape;   // the exchange is built into the block kernel only
        // column groups: block index = row_block * cols + column
        const int64_t n_amax = (rows / brows) * cols;
        zero_floats_kernel<<<(int)((n_amax + 255) / 256 < 1024 ? (n_amax + 255) / 256 : 1024), 256, 0, st>>>(block_amax, n_amax);
        int rows_per_cta = 256;
        if (rows_per_cta > brows) rows_per_cta = brows;
        dim3 grid((unsigned)((cols_vec + 31) / 32), (unsigned)(rows / brows),
                  (unsigned)((brows + rows_per_cta - 1) / rows_per_cta));
        if (is_fp32) amax_nnz_colgroups_kernel<Fp32><<<grid, kThreads, 0, st>>>(static_cast<const float4*>(in), cols_vec, brows, rows_per_cta, block_amax, ws);
        else amax_nnz_colgroups_kernel<Bf16><<<grid, kThreads, 0, st>>>(static_cast<const uint4*>(in), cols_vec, brows, rows_per_cta, block_amax, ws);
        return check_launch();
    }
    if (bcols % epv) return kErrUnsupportedShape;
    const int bcols_vec = bcols / epv;
    const int64_t bx = cols / bcols, nb = bx * (rows / brows);
    if (nb > 0x7FFFFFFF) return kErrTooLarge;
    if (brows == 1 && bcols_vec % kFlatChunkVec == 0 && bcols_vec / kFlatChunkVec <= 4096) {
        if (fuse && fuse->enabled) return kErrUnsupportedShape;
        constexpr int kRing = kFlatWarps * kFlatStages * kFlatChunkVec * 16;
        static SmemOptIn opt32, opt16;
        if (!(is_fp32 ? opt32(amax_nnz_runs_kernel<Fp32>, kRing) : opt16(amax_nnz_runs_kernel<Bf16>, kRing))) return kErrLaunch;
        const unsigned grid = (unsigned)((nb + kFlatWarps - 1) / kFlatWarps);
        const int cpb = bcols_vec / kFlatChunkVec;
        if (is_fp32) amax_nnz_runs_kernel<Fp32><<<grid, kThreads, kRing, st>>>(static_cast<const float4*>(in), cpb, nb, block_amax, ws);
        else amax_nnz_runs_kernel<Bf16><<<grid, kThreads, kRing, st>>>(static_cast<const uint4*>(in), cpb, nb, block_amax, ws);
        return check_launch();
    }
    int w_shift = 0;
    while ((2 << w_shift) <= bcols_vec && (2 << w_shift) <= kThreads) ++w_shift;  // largest power of two <= min(bcols_vec, 256)
    PeerFuse pf{};
    if (fuse) pf = *fuse;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)nb); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    const cudaError_t e = is_fp32
        ? cudaLaunchKernelEx(&cfg, amax_nnz_blocks_kernel<Fp32>, static_cast<const float4*>(in), cols_vec, brows, bcols_vec, bx, w_shift, block_amax, ws, pf)
        : cudaLaunchKernelEx(&cfg, amax_nnz_blocks_kernel<Bf16>, static_cast<const uint4*>(in), cols_vec, brows, bcols_vec, bx, w_shift, block_amax, ws, pf);
    if (e != cudaSuccess) { cudaGetLastError(); return kErrLaunch; }
    return check_launch();
}

}  // namespace morb
