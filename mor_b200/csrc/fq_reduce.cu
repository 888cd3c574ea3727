// amax / non-zero reductions (ref: 951-1049, 1459-1631).  max and integer sums are
// order-independent, so these kernels are free to use any traversal: 16-byte loads,
// warp shuffles, one shared-memory step per CTA, and one atomicMax / atomicAdd per CTA
// into the workspace scalars (the bit pattern of a non-negative float orders like an
// unsigned integer).  NaNs are ignored by fmaxf and never counted, as in the reference.
#include "kernels.cuh"

namespace morb {

namespace {

constexpr int kThreads = 256;

template <typename T>
__device__ __forceinline__ void vec_amax_nnz(const typename T::vec_t& v, float& amax, int& nnz) {
#pragma unroll
    for (int k = 0; k < T::kWordsPerVec; ++k) {
        float hi, lo;
        T::unpack(v, k, hi, lo);
        const float ah = fabsf(hi), al = fabsf(lo);
        amax = fmaxf(amax, fmaxf(ah, al));
        nnz += (ah > 0.0f) + (al > 0.0f);
    }
}

// CTA-wide combine; returns the totals in thread 0.
__device__ __forceinline__ void cta_amax_nnz(float& amax, int& nnz) {
    __shared__ float s_a[32];
    __shared__ int s_n[32];
    amax = warp_max(amax);
    nnz = warp_sum_int(nnz);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { s_a[wid] = amax; s_n[wid] = nnz; }
    __syncthreads();
    if (wid == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        amax = lane < nw ? s_a[lane] : 0.0f;
        nnz = lane < nw ? s_n[lane] : 0;
        amax = warp_max(amax);
        nnz = warp_sum_int(nnz);
    }
    __syncthreads();
}

__global__ void zero_scalars_kernel(ScalarsWs* ws) {
    ws->gamax_bits = 0u; ws->fallback = 0; ws->gnnz = 0ull; ws->gerr = 0.0f; ws->meta = 0;
    ws->pad[0] = ws->pad[1] = 0u;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) amax_nnz_flat_kernel(const typename T::vec_t* __restrict__ in,
                                                                 int64_t nvec, int64_t n_tail_elems,
                                                                 ScalarsWs* __restrict__ ws) {
    float amax = 0.0f;
    int nnz = 0;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t gtid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    for (int64_t i = gtid; i < nvec; i += stride * 4) {
        typename T::vec_t v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i + u * stride < nvec) v[u] = ld_keep(in + i + u * stride);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i + u * stride < nvec) vec_amax_nnz<T>(v[u], amax, nnz);
    }
    if (gtid < n_tail_elems) {
        float a;
        if constexpr (T::kBytesPerElem == 2) a = fabsf(u2f((uint32_t)reinterpret_cast<const uint16_t*>(in + nvec)[gtid] << 16));
        else a = fabsf(reinterpret_cast<const float*>(in + nvec)[gtid]);
        amax = fmaxf(amax, a);
        nnz += a > 0.0f;
    }
    cta_amax_nnz(amax, nnz);
    if (threadIdx.x == 0) {
        atomicMax(&ws->gamax_bits, f2u(amax));
        if (nnz) atomicAdd(&ws->gnnz, (unsigned long long)nnz);
    }
}

// One CTA per (brows x bcols) block; bcols is a multiple of the 16-byte vector width
// and rows are 16-byte aligned (checked by the caller).
template <typename T>
__global__ void __launch_bounds__(kThreads) amax_nnz_blocks_kernel(const typename T::vec_t* __restrict__ in,
                                                                   int64_t cols_vec, int brows, int bcols_vec,
                                                                   int64_t blocks_x, float* __restrict__ block_amax,
                                                                   ScalarsWs* __restrict__ ws) {
    const int64_t b = blockIdx.x;
    const int64_t r0 = (b / blocks_x) * brows, c0 = (b % blocks_x) * bcols_vec;
    float amax = 0.0f;
    int nnz = 0;
    const int n = brows * bcols_vec;
    for (int i = threadIdx.x; i < n; i += kThreads * 4) {
        typename T::vec_t v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int j = i + u * kThreads;
            if (j < n) v[u] = ld_keep(in + (r0 + j / bcols_vec) * cols_vec + c0 + j % bcols_vec);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i + u * kThreads < n) vec_amax_nnz<T>(v[u], amax, nnz);
    }
    cta_amax_nnz(amax, nnz);
    if (threadIdx.x == 0) {
        block_amax[b] = amax;
        atomicMax(&ws->gamax_bits, f2u(amax));
        if (nnz) atomicAdd(&ws->gnnz, (unsigned long long)nnz);
    }
}

// Row groups (1 x k) with k smaller than a CTA's worth: grid-stride over vectors, a
// group is k / elems-per-vector consecutive lanes (a power of two <= 32), combined with
// xor shuffles.  Lane 0 of each group writes the group's amax.
template <typename T>
__global__ void __launch_bounds__(kThreads) amax_nnz_rowgroups_kernel(const typename T::vec_t* __restrict__ in,
                                                                      int64_t nvec, int lanes_per_group,
                                                                      float* __restrict__ block_amax,
                                                                      ScalarsWs* __restrict__ ws) {
    float amax = 0.0f;
    int nnz = 0;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    // nvec is a multiple of 32 (cols is a multiple of 128 elements per row at least)
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += stride) {
        const typename T::vec_t v = ld_keep(in + i);
        float a = 0.0f;
        vec_amax_nnz<T>(v, a, nnz);
        amax = fmaxf(amax, a);
        for (int o = lanes_per_group >> 1; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
        if ((threadIdx.x & (lanes_per_group - 1)) == 0) block_amax[i / lanes_per_group] = a;
    }
    cta_amax_nnz(amax, nnz);
    if (threadIdx.x == 0) {
        atomicMax(&ws->gamax_bits, f2u(amax));
        if (nnz) atomicAdd(&ws->gnnz, (unsigned long long)nnz);
    }
}

// Column groups (k x 1): every thread owns one 16-byte column strip and walks down the
// k rows of its block; per-column maxima go straight to block_amax.
template <typename T>
__global__ void __launch_bounds__(kThreads) amax_nnz_colgroups_kernel(const typename T::vec_t* __restrict__ in,
                                                                      int64_t cols_vec, int brows, int rows_per_cta,
                                                                      float* __restrict__ block_amax,
                                                                      ScalarsWs* __restrict__ ws) {
    constexpr int EPV = 16 / T::kBytesPerElem;
    const int64_t cv = (int64_t)blockIdx.x * kThreads + threadIdx.x;     // vector column
    const int64_t rb = blockIdx.y;                                       // row block
    const int seg = blockIdx.z;                                          // slice of the k rows
    float cmax[EPV];
#pragma unroll
    for (int e = 0; e < EPV; ++e) cmax[e] = 0.0f;
    float amax = 0.0f;
    int nnz = 0;
    if (cv < cols_vec) {
        const int64_t r_begin = rb * brows + (int64_t)seg * rows_per_cta;
        int64_t r_end = r_begin + rows_per_cta;
        if (r_end > (rb + 1) * (int64_t)brows) r_end = (rb + 1) * (int64_t)brows;
        for (int64_t r = r_begin; r < r_end; ++r) {
            const typename T::vec_t v = ld_keep(in + r * cols_vec + cv);
#pragma unroll
            for (int k = 0; k < T::kWordsPerVec; ++k) {
                float hi, lo;
                T::unpack(v, k, hi, lo);
                const float ah = fabsf(hi), al = fabsf(lo);
                cmax[2 * k] = fmaxf(cmax[2 * k], al);
                cmax[2 * k + 1] = fmaxf(cmax[2 * k + 1], ah);
                nnz += (ah > 0.0f) + (al > 0.0f);
            }
        }
#pragma unroll
        for (int e = 0; e < EPV; ++e) {
            amax = fmaxf(amax, cmax[e]);
            atomicMax(reinterpret_cast<uint32_t*>(block_amax) + rb * cols_vec * EPV + cv * EPV + e, f2u(cmax[e]));
        }
    }
    cta_amax_nnz(amax, nnz);
    if (threadIdx.x == 0) {
        atomicMax(&ws->gamax_bits, f2u(amax));
        if (nnz) atomicAdd(&ws->gnnz, (unsigned long long)nnz);
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
    int64_t want = (nvec + kThreads * 4 - 1) / (kThreads * 4);
    const int64_t cap = (int64_t)sm_count() * 8;
    if (want > cap) want = cap;
    if (want < 1) want = 1;
    if (is_fp32) amax_nnz_flat_kernel<Fp32><<<(int)want, kThreads, 0, st>>>(static_cast<const float4*>(in), nvec, tail, ws);
    else amax_nnz_flat_kernel<Bf16><<<(int)want, kThreads, 0, st>>>(static_cast<const uint4*>(in), nvec, tail, ws);
    return check_launch();
}

int launch_amax_nnz_blocks(const void* in, int is_fp32, int64_t rows, int64_t cols, int brows, int bcols,
                           float* block_amax, ScalarsWs* ws, cudaStream_t st) {
    const int epv = is_fp32 ? 4 : 8;
    if (cols % epv) return kErrUnsupportedShape;
    const int64_t cols_vec = cols / epv;
    if (brows == 1 && bcols < 32 * epv) {
        // small row groups: a group is a power-of-two number of lanes
        if (bcols % epv) return kErrUnsupportedShape;
        const int lpg = bcols / epv;
        if (lpg & (lpg - 1)) return kErrUnsupportedShape;
        const int64_t nvec = rows * cols_vec;
        if (nvec % 32) return kErrUnsupportedShape;
        int64_t want = (nvec + kThreads - 1) / kThreads;
        const int64_t cap = (int64_t)sm_count() * 8;
        if (want > cap) want = cap;
        if (is_fp32) amax_nnz_rowgroups_kernel<Fp32><<<(int)want, kThreads, 0, st>>>(static_cast<const float4*>(in), nvec, lpg, block_amax, ws);
        else amax_nnz_rowgroups_kernel<Bf16><<<(int)want, kThreads, 0, st>>>(static_cast<const uint4*>(in), nvec, lpg, block_amax, ws);
        return check_launch();
    }
    if (bcols == 1) {
        // column groups: block index = row_block * cols + column
        const int64_t n_amax = (rows / brows) * cols;
        zero_floats_kernel<<<(int)((n_amax + 255) / 256 < 1024 ? (n_amax + 255) / 256 : 1024), 256, 0, st>>>(block_amax, n_amax);
        int rows_per_cta = 256;
        if (rows_per_cta > brows) rows_per_cta = brows;
        dim3 grid((unsigned)((cols_vec + kThreads - 1) / kThreads), (unsigned)(rows / brows),
                  (unsigned)((brows + rows_per_cta - 1) / rows_per_cta));
        if (is_fp32) amax_nnz_colgroups_kernel<Fp32><<<grid, kThreads, 0, st>>>(static_cast<const float4*>(in), cols_vec, brows, rows_per_cta, block_amax, ws);
        else amax_nnz_colgroups_kernel<Bf16><<<grid, kThreads, 0, st>>>(static_cast<const uint4*>(in), cols_vec, brows, rows_per_cta, block_amax, ws);
        return check_launch();
    }
    if (bcols % epv) return kErrUnsupportedShape;
    const int64_t bx = cols / bcols, nb = bx * (rows / brows);
    if (nb > 0x7FFFFFFF) return kErrTooLarge;
    if (is_fp32) amax_nnz_blocks_kernel<Fp32><<<(unsigned)nb, kThreads, 0, st>>>(static_cast<const float4*>(in), cols_vec, brows, bcols / epv, bx, block_amax, ws);
    else amax_nnz_blocks_kernel<Bf16><<<(unsigned)nb, kThreads, 0, st>>>(static_cast<const uint4*>(in), cols_vec, brows, bcols / epv, bx, block_amax, ws);
    return check_launch();
}

}  // namespace morb
