// TMA tile loads (cp.async.bulk.tensor) and the mbarrier they complete on: device helpers
// and the host-side tensor-map encoder shared by the tile kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace morb {

constexpr uint32_t kSpinLimit = 1u << 22;  // bounded mbarrier wait; a tile that never arrives is reported, not awaited

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// returns false if the barrier did not complete within the spin limit
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}


// untiled bulk copy global -> shared (16-byte aligned addresses, size a multiple of 16)
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// untiled bulk copy shared -> global; the issuing thread commits it to a bulk group and later
// waits until the group's shared-memory reads are done (the buffer may then be reused or freed)
__device__ __forceinline__ void bulk_store(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_reads() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// orders a thread's ordinary shared-memory writes before later reads by the copy engine
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// A warp's private stream of fixed-size chunks of a contiguous global array through
// shared memory: STAGES buffers, one mbarrier each, bulk copies issued by lane 0.  The
// warp takes chunks first, first + step, ...; while it works on one, the next STAGES - 1
// are on their way, whatever the register budget of the kernel.  Every wait is bounded:
// if a copy does not arrive the stream turns itself off for good (`ok` false) and the
// caller reads the data with ordinary loads instead; drain() then gives the copies still
// in flight a last bounded chance to land before the shared memory is handed on.
template <int STAGES, int CHUNK_BYTES>
struct WarpStream {
    uint8_t* buf;        // STAGES * CHUNK_BYTES of shared memory owned by this warp
    uint64_t* bars;      // STAGES barriers owned by this warp
    const uint8_t* src;
    int64_t total_bytes;
    int64_t step;        // distance between this warp's chunks, in chunks
    uint32_t pending;    // bit s: a copy into stage s has been issued and not yet seen complete
    uint32_t phase;      // bit s: parity that copy will flip
    bool ok;

    __device__ __forceinline__ void issue(int64_t chunk, int s) {  // lane 0
        const int64_t off = chunk * CHUNK_BYTES;
        if (off >= total_bytes) return;
        const int64_t left = total_bytes - off;
        const uint32_t bytes = left < CHUNK_BYTES ? (uint32_t)left : (uint32_t)CHUNK_BYTES;
        mbar_expect_tx(&bars[s], bytes);
        bulk_load(buf + s * CHUNK_BYTES, src + off, bytes, &bars[s]);
    }
    __device__ __forceinline__ void start(uint8_t* b, uint64_t* br, const void* s_, int64_t bytes, int64_t first,
                                          int64_t step_) {
        buf = b; bars = br; src = static_cast<const uint8_t*>(s_); total_bytes = bytes; step = step_;
        pending = 0u; phase = 0u; ok = true;
        const int lane = threadIdx.x & 31;
        if (lane == 0) {
#pragma unroll
            for (int s = 0; s < STAGES; ++s) mbar_init(&bars[s], 1);
        }
        __syncwarp();
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            const int64_t c = first + s * step;
            if (c * CHUNK_BYTES < total_bytes) {
                if (lane == 0) issue(c, s);
                pending |= 1u << s;
            }
        }
    }
    // wait for the chunk in stage s; false (warp-uniform, and from then on always) if it did not arrive
    __device__ __forceinline__ bool acquire(int s) {
        if (!ok) return false;
        const bool mine = mbar_wait_bounded(&bars[s], (phase >> s) & 1u);
        if (__all_sync(0xFFFFFFFFu, mine)) {
            pending &= ~(1u << s);
            phase ^= 1u << s;
            return true;
        }
        ok = false;
        return false;
    }
    __device__ __forceinline__ const uint8_t* stage(int s) const { return buf + s * CHUNK_BYTES; }
    // every lane is done with stage s: refill it with chunk `next`
    __device__ __forceinline__ void release(int s, int64_t next) {
        __syncwarp();
        if (ok && next * CHUNK_BYTES < total_bytes) {
            if ((threadIdx.x & 31) == 0) issue(next, s);
            pending |= 1u << s;
        }
    }
    __device__ __forceinline__ void drain() {
#pragma unroll
        for (int s = 0; s < STAGES; ++s)
            if (pending & (1u << s)) mbar_wait_bounded(&bars[s], (phase >> s) & 1u);
    }
};

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
        if (qres != cudaDriverEntryPointSuccess) return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Row-major [rows, cols] tensor of 2- or 4-byte elements, boxes of box_cols x box_rows
// elements, no swizzle.  box_cols * elem_bytes and cols * elem_bytes must be multiples of 16.
inline bool make_tile_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int elem_bytes,
                          int box_cols, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)cols * (cuuint64_t)elem_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estride[2] = {1, 1};
    return fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
              const_cast<void*>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace morb
