// Peer exchange of the row-sharded pipeline over NVLink (no reference counterpart: the
// reference is single-GPU).  Replaces the two scalar all-reduces and the all-gather of the
// per-block error sums by plain stores into buffers that every rank maps from its peers,
// completed by epoch flags:
//
//   scalars  (between the slab amax kernel and the cast kernel)  one warp, lane p for rank p:
//            stores this rank's (amax, nnz) into the peer's slot, fences, stores the epoch,
//            then waits for the epoch in its own slot p; max / sum over the slots;
//   errors   (between the cast kernel and the ordered sum)  a copy kernel stores the slab's
//            error sums into every rank's gathered array; one warp then stores the epoch
//            flags and waits for those of the other ranks.
//
// Only plain peer stores and local loads are used (no multicast, no multimem); slots and
// arrays alternate between two copies by epoch parity, which is enough because a rank can
// be at most one call ahead of the slowest one.  Every wait is bounded: after the limit the
// kernel records the time-out in the workspace head (the call then reports meta = -1) and
// returns, so a lost peer cannot hang the GPU.
#include "kernels.cuh"
#include "p2p.cuh"

namespace morb {

namespace {

// polls of a wait, x 200 ns of back-off: several seconds by default (ranks start a first call unevenly)
uint32_t g_spin_limit = 1u << 25;

// the same exchange as a kernel of its own
__global__ void p2p_exchange_scalars_kernel(ScalarsWs* __restrict__ ws, unsigned char* __restrict__ mine, PeerPtrs peers,
                                            int rank, int world, uint32_t epoch, float* __restrict__ gamax_out,
                                            long long* __restrict__ gnnz_out, uint32_t limit) {
    // the cast kernel behind this one may start now: it requests its tiles and then waits for this kernel to finish
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // this kernel itself may have been launched ahead of the end of the amax kernel: wait for its scalars
    asm volatile("griddepcontrol.wait;" ::: "memory");
    exchange_scalars_warp(ws, mine, peers, rank, world, epoch, gamax_out, gnnz_out, limit);
}

__global__ void __launch_bounds__(256) p2p_push_errors_kernel(const float* __restrict__ local_err, int64_t n_err,
                                                             PeerPtrs peers, int rank, int world, uint32_t epoch) {
    const int64_t stride = (int64_t)gridDim.x * 256;
    const size_t base = kErrOffset + ((size_t)(epoch & 1u) * world + rank) * (size_t)n_err * sizeof(float);
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n_err; i += stride) {
        const float v = local_err[i];
        for (int p = 0; p < world; ++p) reinterpret_cast<float*>(peers.p[p] + base)[i] = v;
    }
}
// launched behind the copy on the same stream: the copy's stores are complete when this starts.
// Tells every rank that this rank's error sums are in place, then waits for theirs.
__global__ void p2p_flag_wait_errors_kernel(const unsigned char* __restrict__ mine, PeerPtrs peers, int rank, int world,
                                            uint32_t epoch, ScalarsWs* __restrict__ ws, uint32_t limit) {
    const int p = threadIdx.x;
    const uint32_t par = epoch & 1u;
    bool ok = true;
    if (p < world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t*>(peers.p[p] + kFlagOffset) + par * kMaxWorld + rank, epoch);
        ok = wait_epoch(reinterpret_cast<const uint32_t*>(mine + kFlagOffset) + par * kMaxWorld + p, epoch, limit);
    }
    if (!__all_sync(0xFFFFFFFFu, ok) && p == 0) atomicOr(&ws->load_timeout, 1u);
}

bool fill_peers_impl(PeerPtrs& pp, void* const* peer_bufs, int world) {
    if (!peer_bufs || world < 1 || world > kMaxWorld) return false;
    for (int i = 0; i < kMaxWorld; ++i) pp.p[i] = nullptr;
    for (int i = 0; i < world; ++i) {
        if (!peer_bufs[i] || (reinterpret_cast<uintptr_t>(peer_bufs[i]) & 255u)) return false;
        pp.p[i] = static_cast<unsigned char*>(peer_bufs[i]);
    }
    return true;
}

}  // namespace

void p2p_set_wait_limit(uint32_t polls) { g_spin_limit = polls ? polls : 1u; }
uint32_t p2p_wait_limit() { return g_spin_limit; }
bool p2p_fill_peers(PeerPtrs& pp, void* const* peer_bufs, int world) { return fill_peers_impl(pp, peer_bufs, world); }

size_t p2p_buffer_bytes(int world, int64_t n_err) {
    if (world < 1 || world > kMaxWorld || n_err < 1) return 0;
    return (kErrOffset + 2 * (size_t)world * (size_t)n_err * sizeof(float) + 255) & ~size_t(255);
}
size_t p2p_error_offset(int world, int64_t n_err, uint32_t epoch) {
    return kErrOffset + (size_t)(epoch & 1u) * (size_t)world * (size_t)n_err * sizeof(float);
}

int launch_p2p_exchange_scalars(ScalarsWs* ws, void* mine, void* const* peer_bufs, int rank, int world, uint32_t epoch,
                                float* gamax_out, long long* gnnz_out, cudaStream_t st) {
    PeerPtrs pp;
    if (!ws || !mine || !gamax_out || !gnnz_out || !fill_peers_impl(pp, peer_bufs, world) || rank < 0 || rank >= world)
        return kErrInvalidArgument;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1); cfg.blockDim = dim3(32); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, p2p_exchange_scalars_kernel, ws, static_cast<unsigned char*>(mine), pp, rank, world, epoch,
                           gamax_out, gnnz_out, g_spin_limit) != cudaSuccess) { cudaGetLastError(); return kErrLaunch; }
    return check_launch();
}
int launch_p2p_exchange_errors(const float* local_err, int64_t n_err, const void* mine, void* const* peer_bufs, int rank,
                               int world, uint32_t epoch, ScalarsWs* ws, cudaStream_t st) {
    PeerPtrs pp;
    if (!local_err || n_err < 1 || !mine || !ws || !fill_peers_impl(pp, peer_bufs, world) || rank < 0 || rank >= world)
        return kErrInvalidArgument;
    int64_t grid = (n_err + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 4;
    if (grid > cap) grid = cap;
    p2p_push_errors_kernel<<<(unsigned)grid, 256, 0, st>>>(local_err, n_err, pp, rank, world, epoch);
    const int rc = check_launch();
    if (rc) return rc;
    p2p_flag_wait_errors_kernel<<<1, 32, 0, st>>>(static_cast<const unsigned char*>(mine), pp, rank, world, epoch, ws, g_spin_limit);
    return check_launch();
}

}  // namespace morb
