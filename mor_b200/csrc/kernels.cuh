// Host-side launch functions of libmor_b200, one per kernel family.  Each returns a
// status code (common.cuh) and never synchronises, allocates or throws.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <cstdlib>

#include "common.cuh"

namespace morb {

int sm_count();                 // SMs of the current device (cached per device)
int check_launch();

// Launch as a programmatic dependent of the kernel before it in the stream: the grid may become resident once every
// CTA of that kernel has executed griddepcontrol.launch_dependents (or exited); what it reads from earlier kernels it
// reads after its own griddepcontrol.wait, which returns when the kernel before it has completed.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }             // cudaGetLastError() -> status code
// test switches (mor_b200_debug_kernel_selection)
bool force_generic();           // skip the TMA-staged tile kernels and the single-pass group kernels
bool resident_disabled();       // skip the single-launch kernel for tensors that fit in shared memory
void set_kernel_selection(int mask);

// Opt-in to more than 48 KiB of dynamic shared memory.  The attribute belongs to a (kernel,
// device) pair, so each launch site keeps one of these and asks it before every launch: the
// runtime call is made once per device, with that device current.
struct SmemOptIn {
    unsigned char done[64] = {};
    template <typename K>
    bool operator()(K kernel, int bytes) {
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
        if (done[dev]) return true;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
        done[dev] = 1;
        return true;
    }
};

// ---- fq_elementwise.cu: one scale for the whole tensor, or none ------------------
// fake_quantize CURRENT_SCALING modes and the BF16 pass-through (ref: 825-844).
int launch_cast_uniform(const void* in, void* out, int64_t n_elems, int fmt, int sf_type, float scale,
                        int32_t* meta, int64_t n_meta, int32_t meta_code, cudaStream_t st);
int launch_copy(const void* in, void* out, int64_t n_bytes, int32_t* meta, int64_t n_meta, int32_t meta_code,
                cudaStream_t st);
// E4M3 bytes + one binary32 scale per block (strategies 1, 3, 4), from the block amax left by launch_amax_nnz_blocks
int launch_quantize_scaled(const void* in, int is_fp32, uint8_t* payload, float* scales, float* gamax_out, int64_t rows,
                           int64_t cols, int brows, int bcols, int ss, const float* block_amax, int64_t n_blocks,
                           const uint32_t* gamax_bits, const float* ext_gamax, cudaStream_t st);
// test operators (ref: 854-875), binary32 in/out
int launch_quant_dequant(const float* in, float* out, int64_t n, int fmt, cudaStream_t st);
int launch_e4m3_e8_scale(const float* in, float* out, int64_t n, int rne, cudaStream_t st);
// E8Mx cast with the scale derived from a device-resident amax (ref: 1335-1428)
int launch_e8mx_cast(const void* in, void* out, int64_t n_elems, int qtype, int strategy,
                     const uint32_t* gamax_bits, cudaStream_t st);

// ---- fq_reduce.cu: amax / non-zero reductions ------------------------------------
// Every workspace starts with a head of kWsHeadBytes: the scalars below in the first 256
// bytes, then room for the 1024 partial sums of a long error array (launch_finalize).
constexpr size_t kChainSumsOffset = 256;
constexpr size_t kWsHeadBytes = kChainSumsOffset + 1024 * sizeof(float);
struct ScalarsWs {              // 40 bytes, zeroed by launch_zero_scalars
    uint32_t gamax_bits;        // max |x| as the bit pattern of a non-negative float
    int32_t fallback;           // 1 when the tensor-level BF16 fallback fired
    unsigned long long gnnz;    // count of non-zero elements
    float gerr;                 // ordered sum of the block errors
    int32_t meta;
    uint32_t div_unsafe;        // a non-zero bf16 magnitude below 2^-90 was seen: take the IEEE division
    uint32_t load_timeout;      // a bounded wait (TMA tile load, grid barrier, peer flag) ran out
    uint32_t bar[2];            // arrival counters of the single-launch kernel's two grid barriers
};
int launch_zero_scalars(ScalarsWs* ws, cudaStream_t st);
// amax and nnz of a flat tensor (phase 1 of e8mx and of the row-sharded pipeline)
int launch_amax_nnz_flat(const void* in, int is_fp32, int64_t n_elems, ScalarsWs* ws, cudaStream_t st);
// per-block amax (brows x bcols blocks, natural row-major block index) + tensor amax/nnz
// `fuse` (may be null): the last CTA also exchanges the slab's amax and count with the other ranks (p2p.cuh);
// kErrUnsupportedShape, with nothing launched, for block shapes whose kernel has no such exchange
struct PeerFuse;
int launch_amax_nnz_blocks(const void* in, int is_fp32, int64_t rows, int64_t cols, int brows, int bcols,
                           float* block_amax, ScalarsWs* ws, cudaStream_t st, const PeerFuse* fuse = nullptr);

// ---- fq_scaling.cu: the amax -> error+cast -> ordered error sum -> fallback pipeline
struct ScalingArgs {
    const void* in;
    void* out;
    int is_fp32;
    int64_t rows, cols;
    int brows, bcols;
    float threshold;
    int ss_mode;
    float* block_amax;          // workspace, one per block
    float* block_err;           // workspace, one per virtual CTA of the reference
    int64_t n_err;              // entries of block_err
    int err_slot_stride;        // the reference stores entry i at slot i * stride of its array
    ScalarsWs* ws;
    const float* ext_gamax;     // optional device pointer: amax of the whole (sharded) tensor
    int early_launch;           // 1: the 128 x 128 tile kernel may start before the previous kernel of the stream has
                                // finished (it waits for it before reading anything that kernel writes)
    void* out_t;                // optional: the output transposed, [cols, rows] (single-pass 128 x 128 tile kernel only)
    int scan_blocks;            // 1: single pass -- the cast kernel takes each block's amax from the tile it
                                // has staged and publishes the tensor's amax / non-zero count itself
                                // (ext_gamax then is the amax of an earlier step: delayed scaling)
};
int launch_block_err_cast(const ScalingArgs& a, bool store, bool only_if_not_fallback, cudaStream_t st);
int launch_rowgroup_err_cast(const ScalingArgs& a, bool store, bool only_if_not_fallback, cudaStream_t st);
int launch_colgroup_err_cast(const ScalingArgs& a, bool store, bool only_if_not_fallback, cudaStream_t st);
int launch_finalize(const ScalingArgs& a, const long long* ext_nnz, int32_t* meta, float* gamax, void* gnnz,
                    int nnz_is_i64, float* gerr, cudaStream_t st);
int launch_fallback_copy(const ScalingArgs& a, cudaStream_t st);
int launch_fallback_transpose(const ScalingArgs& a, cudaStream_t st);   // out_t := in transposed, if the tensor stays BF16

// ---- fq_resident.cu: block scaling on 128 x 128 blocks as one cooperative kernel, for tensors
// that fit in the shared memories of the device (kErrUnsupportedShape otherwise: use the phases above)
int launch_block_resident(const ScalingArgs& a, int32_t* meta, float* gamax, void* gnnz, int nnz_is_i64, float* gerr,
                          cudaStream_t st);
int launch_e8mx_resident(const void* in, void* out, int64_t n_elems, int qtype, int strategy, ScalarsWs* ws,
                         cudaStream_t st);

// ---- fq_block.cu: fake_quantize per-block modes (MoR, block E4M3 / E5M2) ----------
int launch_fq_block(const void* in, void* out, int is_fp32, int32_t* meta, int64_t rows, int64_t cols, int brows,
                    int bcols, float clamp, int quant_mode, int dynamic_range_mode, int sf_type, cudaStream_t st);

// ---- fq_group.cu: single-pass per-group scaling (1 x k groups, MX style) ----------
// narrow-float codes + E8M0 scale bytes of 1 x bcols groups (bf16 input, power-of-two scale)
int launch_quantize_mx(const void* in, void* payload, uint8_t* scales, int64_t rows, int64_t cols, int bcols, int fmt,
                       int pack6, cudaStream_t st);
int launch_fq_group(const void* in, void* out, int is_fp32, float* scales, int32_t* meta, int32_t meta_code,
                    int64_t rows, int64_t cols, int bcols, int fmt, int sf_type, cudaStream_t st);

// ---- p2p.cu: peer exchange of the row-sharded pipeline (plain NVLink stores + epoch flags)
size_t p2p_buffer_bytes(int world, int64_t n_err);
void p2p_set_wait_limit(uint32_t polls);
size_t p2p_error_offset(int world, int64_t n_err, uint32_t epoch);
int launch_p2p_exchange_scalars(ScalarsWs* ws, void* mine, void* const* peer_bufs, int rank, int world, uint32_t epoch,
                                float* gamax_out, long long* gnnz_out, cudaStream_t st);
int launch_p2p_exchange_errors(const float* local_err, int64_t n_err, const void* mine, void* const* peer_bufs, int rank,
                               int world, uint32_t epoch, ScalarsWs* ws, cudaStream_t st);

}  // namespace morb
