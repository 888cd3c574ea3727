// Device side of the peer exchange over NVLink, shared by the exchange kernels (p2p.cu) and by the amax kernel that
// does the exchange itself from its last CTA (fq_reduce.cu).  Only plain peer stores and local loads; every wait is
// bounded.
#pragma once

#include "kernels.cuh"

namespace morb {

constexpr int kMaxWorld = 16;
constexpr size_t kScalOffset = 0, kScalBytes = 2 * kMaxWorld * 32;
constexpr size_t kFlagOffset = kScalBytes, kErrOffset = 2048;

struct ScalSlot {
    uint32_t amax_bits;
    uint32_t pad0;
    unsigned long long nnz;
    uint32_t flag;
    uint32_t pad1[3];
};
static_assert(sizeof(ScalSlot) == 32, "slot size");

struct PeerPtrs {
    unsigned char* p[kMaxWorld];
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool wait_epoch(const uint32_t* flag, uint32_t epoch, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (ld_acquire_sys(flag) == epoch) return true;
        __nanosleep(200);
    }
    return false;
}

// Publish, then gather: one warp, lane p talks to rank p.  Every rank stores before it waits, so the waits cannot
// form a cycle.  The slab's amax and count are read from the workspace head; the tensor's go to gamax_out / gnnz_out.
// A wait that runs out sets the time-out flag of the workspace.
__device__ __forceinline__ void exchange_scalars_warp(ScalarsWs* __restrict__ ws, unsigned char* __restrict__ mine,
                                                      const PeerPtrs& peers, int rank, int world, uint32_t epoch,
                                                      float* __restrict__ gamax_out, long long* __restrict__ gnnz_out,
                                                      uint32_t limit) {
    const int p = threadIdx.x & 31;
    const uint32_t par = epoch & 1u;
    uint32_t amax_bits = 0u;
    unsigned long long nnz = 0ull;
    bool ok = true;
    if (p < world) {
        ScalSlot* out = reinterpret_cast<ScalSlot*>(peers.p[p] + kScalOffset) + par * kMaxWorld + rank;
        out->amax_bits = *reinterpret_cast<volatile uint32_t*>(&ws->gamax_bits);
        out->nnz = *reinterpret_cast<volatile unsigned long long*>(&ws->gnnz);
        __threadfence_system();
        st_release_sys(&out->flag, epoch);
        const ScalSlot* in = reinterpret_cast<const ScalSlot*>(mine + kScalOffset) + par * kMaxWorld + p;
        ok = wait_epoch(&in->flag, epoch, limit);
        if (ok) {
            amax_bits = *reinterpret_cast<const volatile uint32_t*>(&in->amax_bits);
            nnz = *reinterpret_cast<const volatile unsigned long long*>(&in->nnz);
        }
    }
    if (!__all_sync(0xFFFFFFFFu, ok) && p == 0) atomicOr(&ws->load_timeout, 1u);
    amax_bits = __reduce_max_sync(0xFFFFFFFFu, amax_bits);   // non-negative floats order like their bit patterns
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) nnz += __shfl_xor_sync(0xFFFFFFFFu, nnz, o);
    if (p == 0) {
        *gamax_out = u2f(amax_bits);
        *gnnz_out = (long long)nnz;
    }
}

// what the amax kernel needs to do the exchange from its last CTA (enabled == 0: no exchange)
struct PeerFuse {
    unsigned char* mine;
    PeerPtrs peers;
    float* gamax_out;
    long long* gnnz_out;
    int rank, world;
    uint32_t epoch, limit;
    int enabled;
};

bool p2p_fill_peers(PeerPtrs& pp, void* const* peer_bufs, int world);
uint32_t p2p_wait_limit();

}  // namespace morb
