// extern "C" surface of libmor_b200 (include/mor_b200.h): argument validation,
// workspace carving and the fixed kernel sequence of each operator.
#include "../../include/mor_b200.h"

#include <mutex>

#include <cstring>

#include "kernels.cuh"
#include "p2p.cuh"

using namespace morb;

namespace {

constexpr size_t kHead = kWsHeadBytes;  // scalars and partial error sums, ahead of the per-block arrays

inline size_t round256(size_t n) { return (n + 255) & ~size_t(255); }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct Geometry {
    int64_t n_amax;   // per-block amax entries kept in the workspace
    int64_t n_err;    // per-CTA error sums
    int stride;       // slots of the reference's error array per stored sum
    int status;
};

// Shapes accepted by the block pipeline: the reference's 32 x 32-thread CTA strides a
// block in steps of 32 rows x 32 words with no bounds check (ref: 979-987, 1117-1126).
Geometry block_geometry(int64_t rows, int64_t cols, int br, int bc) {
    Geometry g{0, 0, 1, kOk};
    if (rows <= 0 || cols <= 0 || br <= 0 || bc <= 0) { g.status = kErrInvalidArgument; return g; }
    if (rows % br || cols % bc) { g.status = kErrInvalidArgument; return g; }  // ref: 2019-2020
    if (br % 32 || bc % 64) { g.status = kErrUnsupportedShape; return g; }
    g.n_amax = g.n_err = (rows / br) * (cols / bc);
    return g;
}

// ref: 2399-2416, 2499-2511 with grid.y = row blocks (e2m3 fork :2518)
Geometry channel_geometry(int64_t rows, int64_t cols, int br, int bc, int dtype) {
    Geometry g{0, 0, 1, kOk};
    if (rows <= 0 || cols <= 0 || br <= 0 || bc <= 0) { g.status = kErrInvalidArgument; return g; }
    if (!(br == 1 || bc == 1)) { g.status = kErrInvalidArgument; return g; }  // ref: 2501
    if (rows % br || cols % bc || cols % 2) { g.status = kErrInvalidArgument; return g; }
    const int epv = dtype == MOR_B200_FP32 ? 4 : 8;
    if (br == 1) {
        if (bc < 128) {
            if (128 % bc || bc > 64 || bc < epv || cols % 128) { g.status = kErrUnsupportedShape; return g; }
            g.stride = 128 / bc;
            g.n_amax = 0;  // recomputed from the data inside the cast kernel
            g.n_err = rows * (cols / 128);
        } else {
            if (bc % 128) { g.status = kErrUnsupportedShape; return g; }
            g.n_amax = g.n_err = rows * (cols / bc);
        }
    } else {
        if (cols % 64 || br % 16) { g.status = kErrUnsupportedShape; return g; }
        // the column kernels index row blocks with grid.y and slices of a block's rows with grid.z
        if (rows / br > 65535 || (br + 255) / 256 > 65535) { g.status = kErrTooLarge; return g; }
        g.stride = 64;
        g.n_amax = (rows / br) * cols;
        g.n_err = (rows / br) * (cols / 64);
    }
    return g;
}

Geometry geometry(int kind, int64_t rows, int64_t cols, int br, int bc, int dtype) {
    if (kind == MOR_B200_OP_BLOCK_SCALING) return block_geometry(rows, cols, br, bc);
    if (kind == MOR_B200_OP_CHANNEL_SCALING) return channel_geometry(rows, cols, br, bc, dtype);
    return Geometry{0, 0, 1, kErrInvalidArgument};
}

size_t ws_bytes_for(const Geometry& g) { return kHead + round256(4 * (size_t)g.n_amax) + round256(4 * (size_t)g.n_err); }

__global__ void export_scalars_kernel(const ScalarsWs* ws, float* amax_out, long long* nnz_out) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a cast kernel launched behind this one may start
    if (amax_out) *amax_out = u2f(ws->gamax_bits);
    if (nnz_out) *nnz_out = (long long)ws->gnnz;
}

__global__ void __launch_bounds__(256) copy_if_meta3_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                                            int64_t nvec, int64_t tail_bytes,
                                                            const int32_t* __restrict__ meta) {
    if (*meta != 3) return;
    const int64_t stride = (int64_t)gridDim.x * 256;
    const int64_t gtid = (int64_t)blockIdx.x * 256 + threadIdx.x;
    for (int64_t i = gtid; i < nvec; i += stride) out[i] = in[i];
    if (gtid < tail_bytes) reinterpret_cast<uint8_t*>(out + nvec)[gtid] = reinterpret_cast<const uint8_t*>(in + nvec)[gtid];
}

int phase_amax(int kind, const void* in, int dtype, int64_t rows, int64_t cols, int br, int bc, const Geometry& g,
               ScalarsWs* ws, float* block_amax, cudaStream_t st, const PeerFuse* fuse = nullptr) {
    const int is_f32 = dtype == MOR_B200_FP32;
    const bool flat = kind == MOR_B200_OP_CHANNEL_SCALING && g.n_amax == 0;
    // the exchange between ranks is built into the kernel of tall-enough blocks only; checked before anything is launched
    if (fuse && fuse->enabled && (flat || bc == 1 || (br == 1 && (int64_t)bc * (is_f32 ? 4 : 2) % 4096 == 0)))
        return kErrUnsupportedShape;
    int rc = launch_zero_scalars(ws, st);
    if (rc) return rc;
    if (flat) return launch_amax_nnz_flat(in, is_f32, rows * cols, ws, st);
    return launch_amax_nnz_blocks(in, is_f32, rows, cols, br, bc, block_amax, ws, st, fuse);
}

int phase_cast(int kind, const ScalingArgs& a, bool store, bool skip_if_fallback, cudaStream_t st) {
    if (kind == MOR_B200_OP_BLOCK_SCALING) return launch_block_err_cast(a, store, skip_if_fallback, st);
    if (a.brows == 1) return launch_rowgroup_err_cast(a, store, skip_if_fallback, st);
    return launch_colgroup_err_cast(a, store, skip_if_fallback, st);
}

int scaling_op(int kind, const void* in, void* out, int dtype, int64_t rows, int64_t cols, int br, int bc, double thr,
               int ss, int32_t* meta, float* gamax, void* gnnz, int nnz64, float* gerr, void* wsp, size_t wsb,
               void* stream) {
    if (!in || !out || (dtype != MOR_B200_BF16 && dtype != MOR_B200_FP32)) return kErrInvalidArgument;
    if (ss < 1 || ss > 4) return kErrInvalidArgument;  // the reference falls off a switch here (ref: 2120)
    const Geometry g = geometry(kind, rows, cols, br, bc, dtype);
    if (g.status) return g.status;
    if (!aligned16(in) || !aligned16(out)) return kErrUnsupportedShape;
    if (!wsp || wsb < ws_bytes_for(g) || !aligned16(wsp)) return kErrWorkspace;
    auto st = static_cast<cudaStream_t>(stream);
    auto* ws = static_cast<ScalarsWs*>(wsp);
    ScalingArgs a{};
    a.in = in; a.out = out; a.is_fp32 = dtype == MOR_B200_FP32; a.rows = rows; a.cols = cols;
    a.brows = br; a.bcols = bc; a.threshold = (float)thr; a.ss_mode = ss;
    a.block_amax = reinterpret_cast<float*>(static_cast<char*>(wsp) + kHead);
    a.block_err = reinterpret_cast<float*>(static_cast<char*>(wsp) + kHead + round256(4 * (size_t)g.n_amax));
    a.n_err = g.n_err; a.err_slot_stride = g.stride; a.ws = ws; a.ext_gamax = nullptr;
    const bool inplace = in == out;
    // Small tensors (all tiles fit in the shared memories of the device): one cooperative launch that
    // reads the tensor once, whatever the strategy; in place too.
    if (kind == MOR_B200_OP_BLOCK_SCALING && br == 128 && bc == 128) {
        const int rcr = launch_block_resident(a, meta, gamax, gnnz, nnz64, gerr, st);
        if (rcr != kErrUnsupportedShape) return rcr;
    }
    // Strategies 2 and 3 scale a block by its own amax only: on 128 x 128 blocks the tile kernel
    // takes it from the staged tile, and the separate amax pass over the tensor is not needed.
    if (kind == MOR_B200_OP_BLOCK_SCALING && br == 128 && bc == 128 && (ss == 2 || ss == 3) && !inplace) {
        a.scan_blocks = 1;
        int rc1 = launch_zero_scalars(ws, st);
        if (rc1) return rc1;
        rc1 = launch_block_err_cast(a, /*store=*/true, false, st);
        if (rc1 == kOk) {
            rc1 = launch_finalize(a, nullptr, meta, gamax, gnnz, nnz64, gerr, st);
            if (rc1) return rc1;
            return launch_fallback_copy(a, st);
        }
        if (rc1 != kErrUnsupportedShape) return rc1;
        a.scan_blocks = 0;   // no tile path for this tensor: the two-pass form below
    }
    // The same for 1 x k row groups (strategies 2 and 3 again): the cast kernels that recompute a group's amax
    // themselves also publish the tensor's amax and count, and the amax pass is left out.
    if (kind == MOR_B200_OP_CHANNEL_SCALING && br == 1 && (ss == 2 || ss == 3) && !inplace && !force_generic()) {
        a.scan_blocks = 1;
        int rc1 = launch_zero_scalars(ws, st);
        if (rc1) return rc1;
        rc1 = launch_rowgroup_err_cast(a, /*store=*/true, false, st);
        if (rc1 == kOk) {
            rc1 = launch_finalize(a, nullptr, meta, gamax, gnnz, nnz64, gerr, st);
            if (rc1) return rc1;
            return launch_fallback_copy(a, st);
        }
        if (rc1 != kErrUnsupportedShape) return rc1;
        a.scan_blocks = 0;   // no single-pass kernel for this shape: the two-pass form below
    }
    int rc = phase_amax(kind, in, dtype, rows, cols, br, bc, g, ws, a.block_amax, st);
    if (rc) return rc;
    // In place the input must survive until the tensor-level decision is known: sum the
    // errors without storing, decide, then cast only if the tensor is kept in E4M3.
    a.early_launch = 1;   // the tile kernel may become resident, and request its tiles, during the amax kernel's last wave
    rc = phase_cast(kind, a, /*store=*/!inplace, false, st);
    a.early_launch = 0;
    if (rc) return rc;
    rc = launch_finalize(a, nullptr, meta, gamax, gnnz, nnz64, gerr, st);
    if (rc) return rc;
    if (inplace) {
        ScalingArgs b = a;
        b.block_err = a.block_err;  // rewritten with identical values
        return phase_cast(kind, b, /*store=*/true, /*skip_if_fallback=*/true, st);
    }
    return launch_fallback_copy(a, st);
}

// ---- scratch for mor_b200_block_scaling_static ------------------------------------
// Sized for kStaticMaxBlocks blocks: scalar head + one amax and one error sum per block.
// Device memory that every GPU loading this library holds until the process exits.
constexpr int64_t kStaticMaxBlocks = 65536;
constexpr size_t kStaticScratchBytes = kHead + 2 * 4 * (size_t)kStaticMaxBlocks;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code the name g_static_scratch is only a handle for the runtime, not a device
// address; the address each device gave the array is looked up once per device (with
// that device current) and cached.
void* static_scratch_ptr(int* status) {
    static std::mutex mu;
    static void* ptrs[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *status = kErrLaunch; return nullptr; }
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) { *status = kErrLaunch; return nullptr; }
        ptrs[dev] = p;
    }
    *status = kOk;
    return ptrs[dev];
}

}  // namespace

extern "C" {

int mor_b200_version(void) { return 110; }

void mor_b200_debug_kernel_selection(int mask) { set_kernel_selection(mask); }

const char* mor_b200_status_string(int status) {
    switch (status) {
        case kOk: return "ok";
        case kErrInvalidArgument: return "invalid argument";
        case kErrUnsupportedShape: return "unsupported shape or alignment";
        case kErrWorkspace: return "workspace missing, misaligned or too small";
        case kErrLaunch: return "CUDA launch failed";
        case kErrTooLarge: return "too many blocks for one grid";
        case -6: return "tensor has more blocks than the built-in scratch holds (65536); use the workspace form";
        default: return "unknown status";
    }
}

size_t mor_b200_workspace_bytes(int op, int64_t rows, int64_t cols, int br, int bc) {
    if (op == MOR_B200_OP_E8MX || op == MOR_B200_OP_AMAX_NNZ) return kHead;
    // sized for the wider of the two dtypes' geometries (they only differ in which small groups are accepted)
    Geometry g = geometry(op, rows, cols, br, bc, MOR_B200_BF16);
    if (g.status) g = geometry(op, rows, cols, br, bc, MOR_B200_FP32);
    if (g.status) return 0;
    return ws_bytes_for(g);
}

int mor_b200_fake_quantize(const void* in, void* out, int32_t* meta, int dtype, int64_t rows, int64_t cols, int br,
                           int bc, double clamp, int mode, int sf_type, void* stream) {
    if (!in || !out || !meta) return kErrInvalidArgument;
    if (dtype != MOR_B200_BF16 && dtype != MOR_B200_FP32) return kErrInvalidArgument;
    if (rows <= 0 || cols <= 0 || br <= 0 || bc < 2 || mode < 0) return kErrInvalidArgument;
    if (cols % 2 || bc % 2) return kErrInvalidArgument;  // ref: 1767; odd block widths split a packed word
    if (sf_type != kSfFp32 && sf_type != kSfE8) return kErrInvalidArgument;
    const int esz = dtype == MOR_B200_FP32 ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & (2 * esz - 1)) return kErrUnsupportedShape;
    auto st = static_cast<cudaStream_t>(stream);
    const int qm = mode % 10;
    const int dyn = mode / 100 > 0;
    const int64_t gx = (cols / 2 - 1) / (bc / 2) + 1, gy = (rows - 1) / br + 1, n_meta = gx * gy;
    if (qm == 4 || qm == 5) {
        if (dtype != MOR_B200_BF16 || !aligned16(in) || !aligned16(out)) return kErrUnsupportedShape;
        return launch_cast_uniform(in, out, rows * cols, qm == 4 ? kE4M3 : kE5M2, sf_type, (float)clamp, meta, n_meta,
                                   qm == 4 ? 1 : 2, st);
    }
    if (qm != 1 && qm != 2 && qm != 3) {  // ref: 1831: every other code is the BF16 pass-through
        if (!aligned16(in) || !aligned16(out)) return kErrUnsupportedShape;
        return launch_copy(in, out, rows * cols * esz, meta, n_meta, 3, st);
    }
    if (qm == 1 && (int64_t)br * bc > 1024 && (br < 32 || bc < 32)) return kErrUnsupportedShape;  // ref: 1781-1784
    // per-row groups in the fixed-format modes take the single-pass group kernels
    if (qm != 1 && br == 1 && cols % bc == 0 && aligned16(in) && aligned16(out) && !force_generic()) {
        const int rc = launch_fq_group(in, out, dtype == MOR_B200_FP32, nullptr, meta, qm == 2 ? 1 : 2, rows, cols, bc,
                                       qm == 2 ? kE4M3 : kE5M2, sf_type, st);
        if (rc != kErrUnsupportedShape) return rc;
    }
    return launch_fq_block(in, out, dtype == MOR_B200_FP32, meta, rows, cols, br, bc, (float)clamp, qm, dyn, sf_type, st);
}

int mor_b200_quant_dequant(const float* in, float* out, int64_t rows, int64_t cols, int format, void* stream) {
    if (!in || !out || rows <= 0 || cols <= 0) return kErrInvalidArgument;
    return launch_quant_dequant(in, out, rows * cols, format, static_cast<cudaStream_t>(stream));
}

int mor_b200_e4m3_with_e8_scale(const float* in, float* out, int64_t rows, int64_t cols, int rne, void* stream) {
    if (!in || !out || rows <= 0 || cols <= 0) return kErrInvalidArgument;
    return launch_e4m3_e8_scale(in, out, rows * cols, rne, static_cast<cudaStream_t>(stream));
}

int mor_b200_block_scaling(const void* in, void* out, int dtype, int64_t rows, int64_t cols, int br, int bc,
                           double thr, int ss, int32_t* meta, float* gamax, void* gnnz, int nnz64, float* gerr,
                           void* ws, size_t wsb, void* stream) {
    return scaling_op(MOR_B200_OP_BLOCK_SCALING, in, out, dtype, rows, cols, br, bc, thr, ss, meta, gamax, gnnz, nnz64,
                      gerr, ws, wsb, stream);
}

int mor_b200_block_scaling_static(const void* in, void* out, int dtype, int64_t rows, int64_t cols, int br, int bc,
                                  double thr, int ss, int32_t* meta, float* gamax, void* gnnz, int nnz64,
                                  float* gerr, void* stream) {
    const Geometry g = block_geometry(rows, cols, br, bc);
    if (g.status) return g.status;
    if (g.n_amax > kStaticMaxBlocks) return -6;
    int rc = kOk;
    void* ws = static_scratch_ptr(&rc);
    if (rc) return rc;
    // the scalar head is zeroed by the first kernel of every call; the per-block arrays are
    // fully rewritten before they are read, so nothing of the previous call survives
    return scaling_op(MOR_B200_OP_BLOCK_SCALING, in, out, dtype, rows, cols, br, bc, thr, ss, meta, gamax, gnnz, nnz64,
                      gerr, ws, kStaticScratchBytes, stream);
}

int mor_b200_channel_scaling(const void* in, void* out, int dtype, int64_t rows, int64_t cols, int br, int bc,
                             double thr, int ss, int32_t* meta, float* gamax, void* gnnz, int nnz64, float* gerr,
                             void* ws, size_t wsb, void* stream) {
    return scaling_op(MOR_B200_OP_CHANNEL_SCALING, in, out, dtype, rows, cols, br, bc, thr, ss, meta, gamax, gnnz,
                      nnz64, gerr, ws, wsb, stream);
}

int mor_b200_e8mx(const void* in, void* out, int64_t rows, int64_t cols, int qtype, int strategy, void* wsp,
                  size_t wsb, void* stream) {
    if (!in || !out || rows <= 0 || cols <= 0 || cols % 2) return kErrInvalidArgument;
    if (qtype < 1 || qtype > 3) return kErrInvalidArgument;
    if (!aligned16(in) || !aligned16(out)) return kErrUnsupportedShape;
    if (!wsp || wsb < kHead || !aligned16(wsp)) return kErrWorkspace;
    auto st = static_cast<cudaStream_t>(stream);
    auto* ws = static_cast<ScalarsWs*>(wsp);
    // small tensors: one cooperative launch that keeps the tensor in shared memory between the amax and the cast
    int rc = launch_e8mx_resident(in, out, rows * cols, qtype, strategy, ws, st);
    if (rc != kErrUnsupportedShape) return rc;
    rc = launch_zero_scalars(ws, st);
    if (rc) return rc;
    rc = launch_amax_nnz_flat(in, 0, rows * cols, ws, st);
    if (rc) return rc;
    return launch_e8mx_cast(in, out, rows * cols, qtype, strategy, &ws->gamax_bits, st);
}

int mor_b200_fake_quantize_group(const void* in, void* out, float* scales, int dtype, int64_t rows, int64_t cols,
                                 int bc, int format, int sf_type, void* stream) {
    if (!in || !out || rows <= 0 || cols <= 0 || bc <= 0) return kErrInvalidArgument;
    if (dtype != MOR_B200_BF16 && dtype != MOR_B200_FP32) return kErrInvalidArgument;
    if (sf_type != kSfFp32 && sf_type != kSfE8) return kErrInvalidArgument;
    if (cols % bc) return kErrInvalidArgument;
    if (!aligned16(in) || !aligned16(out)) return kErrUnsupportedShape;
    return launch_fq_group(in, out, dtype == MOR_B200_FP32, scales, nullptr, 0, rows, cols, bc, format, sf_type,
                           static_cast<cudaStream_t>(stream));
}

// Single pass with a delayed tensor amax: the scales use `amax_in` (device, e.g. the amax this call
// reported for the previous step's tensor), every block's own amax comes from the staged tile, and
// the tensor's amax / non-zero count / error of THIS call are reported for the next one.
namespace {
int delayed_op(const void* in, void* out, void* out_t, int dtype, int64_t rows, int64_t cols, int br, int bc, double thr, int ss,
               const float* amax_in, int32_t* meta, float* amax_out, void* nnz_out, int nnz64, float* err_out, void* wsp,
               size_t wsb, void* stream);
}  // namespace

int mor_b200_block_scaling_delayed(const void* in, void* out, int dtype, int64_t rows, int64_t cols, int br, int bc,
                                   double thr, int ss, const float* amax_in, int32_t* meta, float* amax_out,
                                   void* nnz_out, int nnz64, float* err_out, void* wsp, size_t wsb, void* stream) {
    if (!out) return kErrInvalidArgument;
    return delayed_op(in, out, nullptr, dtype, rows, cols, br, bc, thr, ss, amax_in, meta, amax_out, nnz_out, nnz64, err_out,
                      wsp, wsb, stream);
}

int mor_b200_block_scaling_delayed_t(const void* in, void* out, void* out_t, int dtype, int64_t rows, int64_t cols, int br,
                                     int bc, double thr, int ss, const float* amax_in, int32_t* meta, float* amax_out,
                                     void* nnz_out, int nnz64, float* err_out, void* wsp, size_t wsb, void* stream) {
    if (!out_t || out_t == in || out_t == out || !aligned16(out_t)) return kErrInvalidArgument;
    return delayed_op(in, out, out_t, dtype, rows, cols, br, bc, thr, ss, amax_in, meta, amax_out, nnz_out, nnz64, err_out,
                      wsp, wsb, stream);
}

namespace {
int delayed_op(const void* in, void* out, void* out_t, int dtype, int64_t rows, int64_t cols, int br, int bc, double thr, int ss,
               const float* amax_in, int32_t* meta, float* amax_out, void* nnz_out, int nnz64, float* err_out, void* wsp,
               size_t wsb, void* stream) {
    if (!in || (!out && !out_t) || !amax_in || (dtype != MOR_B200_BF16 && dtype != MOR_B200_FP32)) return kErrInvalidArgument;
    if (ss < 1 || ss > 4) return kErrInvalidArgument;
    if (br != 128 || bc != 128 || in == out) return kErrUnsupportedShape;   // TMA-staged tiles; the fallback needs the input
    const Geometry g = block_geometry(rows, cols, br, bc);
    if (g.status) return g.status;
    if (!aligned16(in) || (out && !aligned16(out))) return kErrUnsupportedShape;
    if (!wsp || wsb < ws_bytes_for(g) || !aligned16(wsp)) return kErrWorkspace;
    auto st = static_cast<cudaStream_t>(stream);
    auto* ws = static_cast<ScalarsWs*>(wsp);
    ScalingArgs a{};
    a.in = in; a.out = out; a.is_fp32 = dtype == MOR_B200_FP32; a.rows = rows; a.cols = cols;
    a.brows = br; a.bcols = bc; a.threshold = (float)thr; a.ss_mode = ss;
    a.block_amax = reinterpret_cast<float*>(static_cast<char*>(wsp) + kHead);
    a.block_err = reinterpret_cast<float*>(static_cast<char*>(wsp) + kHead + round256(4 * (size_t)g.n_amax));
    a.n_err = g.n_err; a.err_slot_stride = g.stride; a.ws = ws; a.ext_gamax = amax_in; a.scan_blocks = 1; a.out_t = out_t;
    int rc = launch_zero_scalars(ws, st);
    if (rc) return rc;
    rc = launch_block_err_cast(a, /*store=*/true, false, st);
    if (rc) return rc;
    ScalingArgs f = a;
    f.ext_gamax = nullptr;   // report the amax found in this tensor, not the one the scales were built from
    rc = launch_finalize(f, nullptr, meta, amax_out, nnz_out, nnz64, err_out, st);
    if (rc) return rc;
    rc = launch_fallback_copy(a, st);
    if (rc) return rc;
    return launch_fallback_transpose(a, st);
}
}  // namespace

int mor_b200_quantize_mx(const void* in, void* payload, void* scales, int64_t rows, int64_t cols, int bc, int format,
                         void* stream) {
    if (!in || !payload || !scales || rows <= 0 || cols <= 0 || bc <= 0) return kErrInvalidArgument;
    if (cols % bc) return kErrInvalidArgument;
    if (format != kE4M3 && format != kE5M2 && format != kE2M3) return kErrInvalidArgument;
    if (!aligned16(in) || (reinterpret_cast<uintptr_t>(payload) & 7u)) return kErrUnsupportedShape;
    return launch_quantize_mx(in, payload, static_cast<uint8_t*>(scales), rows, cols, bc, format, 0,
                              static_cast<cudaStream_t>(stream));
}
int mor_b200_quantize_mx_fp6(const void* in, void* payload, void* scales, int64_t rows, int64_t cols, int bc,
                             void* stream) {
    if (!in || !payload || !scales || rows <= 0 || cols <= 0 || bc <= 0) return kErrInvalidArgument;
    if (cols % bc) return kErrInvalidArgument;
    if (!aligned16(in) || (reinterpret_cast<uintptr_t>(payload) & 1u)) return kErrUnsupportedShape;
    return launch_quantize_mx(in, payload, static_cast<uint8_t*>(scales), rows, cols, bc, kE2M3, 1,
                              static_cast<cudaStream_t>(stream));
}

int mor_b200_quantize_scaled(const void* in, void* payload, float* scales, int dtype, int64_t rows, int64_t cols, int br,
                             int bc, int ss, const float* amax_in, float* amax_out, void* wsp, size_t wsb, void* stream) {
    if (!in || !payload || !scales || (dtype != MOR_B200_BF16 && dtype != MOR_B200_FP32)) return kErrInvalidArgument;
    if (ss != 1 && ss != 3 && ss != 4) return kErrInvalidArgument;   // strategy 2 is a power of two: mor_b200_quantize_mx
    const int kind = (br == 1 || bc == 1) ? MOR_B200_OP_CHANNEL_SCALING : MOR_B200_OP_BLOCK_SCALING;
    const Geometry g = geometry(kind, rows, cols, br, bc, dtype);
    if (g.status) return g.status;
    if (g.n_amax == 0) return kErrUnsupportedShape;   // 1 x k groups below 128 columns keep no amax array
    if (!aligned16(in) || (reinterpret_cast<uintptr_t>(payload) & 7u) || cols % 8) return kErrUnsupportedShape;
    if (!wsp || wsb < ws_bytes_for(g) || !aligned16(wsp)) return kErrWorkspace;
    auto st = static_cast<cudaStream_t>(stream);
    auto* ws = static_cast<ScalarsWs*>(wsp);
    float* block_amax = reinterpret_cast<float*>(static_cast<char*>(wsp) + kHead);
    const int rc = phase_amax(kind, in, dtype, rows, cols, br, bc, g, ws, block_amax, st);
    if (rc) return rc;
    return launch_quantize_scaled(in, dtype == MOR_B200_FP32, static_cast<uint8_t*>(payload), scales, amax_out, rows, cols,
                                  br, bc, ss, block_amax, g.n_amax, &ws->gamax_bits, amax_in, st);
}

int mor_b200_scaling_amax(int kind, const void* in, int dtype, int64_t rows, int64_t cols, int br, int bc,
                          float* amax_out, int64_t* nnz_out, void* wsp, size_t wsb, void* stream) {
    if (!in || (dtype != MOR_B200_BF16 && dtype != MOR_B200_FP32)) return kErrInvalidArgument;
    const Geometry g = geometry(kind, rows, cols, br, bc, dtype);
    if (g.status) return g.status;
    if (!aligned16(in)) return kErrUnsupportedShape;
    if (!wsp || wsb < ws_bytes_for(g) || !aligned16(wsp)) return kErrWorkspace;
    auto st = static_cast<cudaStream_t>(stream);
    auto* ws = static_cast<ScalarsWs*>(wsp);
    const int rc = phase_amax(kind, in, dtype, rows, cols, br, bc, g, ws, reinterpret_cast<float*>(static_cast<char*>(wsp) + kHead), st);
    if (rc) return rc;
    if (!amax_out && !nnz_out) return kOk;   // the caller takes them from the workspace head (peer exchange)
    export_scalars_kernel<<<1, 1, 0, st>>>(ws, amax_out, reinterpret_cast<long long*>(nnz_out));
    return check_launch();
}

int mor_b200_scaling_amax_p2p(int kind, const void* in, int dtype, int64_t rows, int64_t cols, int br, int bc,
                              void* wsp, size_t wsb, void* my_buf, void* const* peer_bufs, int rank, int world,
                              uint32_t epoch, float* global_amax, int64_t* global_nnz, void* stream) {
    if (!in || !my_buf || !global_amax || !global_nnz || (dtype != MOR_B200_BF16 && dtype != MOR_B200_FP32))
        return kErrInvalidArgument;
    const Geometry g = geometry(kind, rows, cols, br, bc, dtype);
    if (g.status) return g.status;
    if (!aligned16(in)) return kErrUnsupportedShape;
    if (!wsp || wsb < ws_bytes_for(g) || !aligned16(wsp)) return kErrWorkspace;
    PeerFuse pf{};
    if (!p2p_fill_peers(pf.peers, peer_bufs, world) || rank < 0 || rank >= world) return kErrInvalidArgument;
    pf.mine = static_cast<unsigned char*>(my_buf);
    pf.gamax_out = global_amax;
    pf.gnnz_out = reinterpret_cast<long long*>(global_nnz);
    pf.rank = rank; pf.world = world; pf.epoch = epoch; pf.limit = p2p_wait_limit(); pf.enabled = 1;
    return phase_amax(kind, in, dtype, rows, cols, br, bc, g, static_cast<ScalarsWs*>(wsp),
                      reinterpret_cast<float*>(static_cast<char*>(wsp) + kHead), static_cast<cudaStream_t>(stream), &pf);
}

int mor_b200_scaling_cast(int kind, const void* in, void* out, int dtype, int64_t rows, int64_t cols, int br, int bc,
                          int ss, const float* global_amax, float* block_err_out, void* wsp, size_t wsb,
                          void* stream) {
    if (!in || !out || !global_amax || !block_err_out) return kErrInvalidArgument;
    if (dtype != MOR_B200_BF16 && dtype != MOR_B200_FP32) return kErrInvalidArgument;
    if (ss < 1 || ss > 4) return kErrInvalidArgument;
    const Geometry g = geometry(kind, rows, cols, br, bc, dtype);
    if (g.status) return g.status;
    if (!aligned16(in) || !aligned16(out)) return kErrUnsupportedShape;
    if (!wsp || wsb < ws_bytes_for(g) || !aligned16(wsp)) return kErrWorkspace;
    ScalingArgs a{};
    a.in = in; a.out = out; a.is_fp32 = dtype == MOR_B200_FP32; a.rows = rows; a.cols = cols;
    a.brows = br; a.bcols = bc; a.threshold = 0.0f; a.ss_mode = ss;
    a.block_amax = reinterpret_cast<float*>(static_cast<char*>(wsp) + kHead);
    a.block_err = block_err_out;
    a.n_err = g.n_err; a.err_slot_stride = g.stride; a.ws = static_cast<ScalarsWs*>(wsp); a.ext_gamax = global_amax;
    a.early_launch = 1;   // behind the kernel (or collective) that delivers the global amax
    return phase_cast(kind, a, /*store=*/true, false, static_cast<cudaStream_t>(stream));
}

int64_t mor_b200_scaling_num_errors(int kind, int64_t rows, int64_t cols, int br, int bc) {
    Geometry g = geometry(kind, rows, cols, br, bc, MOR_B200_BF16);
    if (g.status) g = geometry(kind, rows, cols, br, bc, MOR_B200_FP32);
    return g.status ? -1 : g.n_err;
}

int mor_b200_scaling_error_stride(int kind, int br, int bc) {
    if (kind == MOR_B200_OP_BLOCK_SCALING) return 1;
    if (kind != MOR_B200_OP_CHANNEL_SCALING) return -1;
    if (br == 1) return (bc < 128 && bc > 0 && 128 % bc == 0) ? 128 / bc : 1;
    return 64;
}

int mor_b200_scaling_finalize(const float* block_err, int64_t n_err, int stride, const int64_t* global_nnz, double thr,
                              int32_t* meta, float* global_error, void* wsp, size_t wsb, void* stream) {
    if (!block_err || n_err <= 0 || !global_nnz || !meta) return kErrInvalidArgument;
    if (stride < 1 || stride > 64 || (stride & (stride - 1))) return kErrInvalidArgument;
    if (!wsp || wsb < kHead || !aligned16(wsp)) return kErrWorkspace;
    ScalingArgs a{};
    a.block_err = const_cast<float*>(block_err);
    a.n_err = n_err; a.err_slot_stride = stride; a.threshold = (float)thr; a.ws = static_cast<ScalarsWs*>(wsp);
    return launch_finalize(a, reinterpret_cast<const long long*>(global_nnz), meta, nullptr, nullptr, 0, global_error,
                           static_cast<cudaStream_t>(stream));
}

int mor_b200_scaling_fallback(const void* in, void* out, int64_t n_bytes, const int32_t* meta, void* stream) {
    if (!in || !out || !meta || n_bytes < 0) return kErrInvalidArgument;
    if (in == out || n_bytes == 0) return kOk;
    if (!aligned16(in) || !aligned16(out)) return kErrUnsupportedShape;
    const int64_t nvec = n_bytes / 16;
    int64_t grid = (nvec + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    copy_if_meta3_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(in), static_cast<uint4*>(out), nvec, n_bytes % 16, meta);
    return check_launch();
}

size_t mor_b200_p2p_bytes(int world, int64_t n_err) { return p2p_buffer_bytes(world, n_err); }
void mor_b200_p2p_set_wait_limit(uint32_t polls) { p2p_set_wait_limit(polls); }
size_t mor_b200_p2p_error_offset(int world, int64_t n_err, uint32_t epoch) { return p2p_error_offset(world, n_err, epoch); }

// The buffer is allocated, exported and opened here, not through the caller's allocator: a peer's
// buffer has to be opened while the CURRENT device is the one whose kernels will store into it
// (cudaIpcOpenMemHandle maps it for that device and enables peer access to its owner).
namespace {
struct DeviceScope {
    int prev = -1;
    bool ok = false;
    explicit DeviceScope(int device) { ok = cudaGetDevice(&prev) == cudaSuccess && cudaSetDevice(device) == cudaSuccess; }
    ~DeviceScope() { if (prev >= 0) cudaSetDevice(prev); }
};
}  // namespace

int mor_b200_p2p_alloc(int device, size_t bytes, void** ptr_out, unsigned char* handle_out) {
    if (device < 0 || bytes == 0 || !ptr_out || !handle_out) return kErrInvalidArgument;
    static_assert(sizeof(cudaIpcMemHandle_t) == MOR_B200_P2P_HANDLE_BYTES, "handle size");
    DeviceScope scope(device);
    if (!scope.ok) return kErrLaunch;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return kErrWorkspace; }
    cudaIpcMemHandle_t h;
    if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
        cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(p);
        return kErrLaunch;
    }
    memcpy(handle_out, &h, sizeof(h));
    *ptr_out = p;
    return kOk;
}
int mor_b200_p2p_open(int device, const unsigned char* handle, void** ptr_out) {
    if (device < 0 || !handle || !ptr_out) return kErrInvalidArgument;
    DeviceScope scope(device);
    if (!scope.ok) return kErrLaunch;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return kErrLaunch; }
    *ptr_out = p;
    return kOk;
}
int mor_b200_p2p_close(int device, void* peer_ptr) {
    if (device < 0 || !peer_ptr) return kErrInvalidArgument;
    DeviceScope scope(device);
    if (!scope.ok) return kErrLaunch;
    if (cudaIpcCloseMemHandle(peer_ptr) != cudaSuccess) { cudaGetLastError(); return kErrLaunch; }
    return kOk;
}
int mor_b200_p2p_free(int device, void* own_ptr) {
    if (device < 0 || !own_ptr) return kErrInvalidArgument;
    DeviceScope scope(device);
    if (!scope.ok) return kErrLaunch;
    if (cudaFree(own_ptr) != cudaSuccess) { cudaGetLastError(); return kErrLaunch; }
    return kOk;
}

int mor_b200_p2p_exchange_scalars(void* wsp, void* my_buf, void* const* peer_bufs, int rank, int world, uint32_t epoch,
                                  float* global_amax, int64_t* global_nnz, void* stream) {
    if (!wsp || !aligned16(wsp)) return kErrWorkspace;
    return launch_p2p_exchange_scalars(static_cast<ScalarsWs*>(wsp), my_buf, peer_bufs, rank, world, epoch, global_amax,
                                       reinterpret_cast<long long*>(global_nnz), static_cast<cudaStream_t>(stream));
}
int mor_b200_p2p_exchange_errors(const float* local_err, int64_t n_err, const void* my_buf, void* const* peer_bufs,
                                 int rank, int world, uint32_t epoch, void* wsp, void* stream) {
    if (!wsp || !aligned16(wsp)) return kErrWorkspace;
    return launch_p2p_exchange_errors(local_err, n_err, my_buf, peer_bufs, rank, world, epoch,
                                      static_cast<ScalarsWs*>(wsp), static_cast<cudaStream_t>(stream));
}

int mor_b200_amax_nnz(const void* in, int dtype, int64_t n, float* amax_out, int64_t* nnz_out, void* wsp, size_t wsb,
                      void* stream) {
    if (!in || n <= 0 || (dtype != MOR_B200_BF16 && dtype != MOR_B200_FP32)) return kErrInvalidArgument;
    if (!aligned16(in)) return kErrUnsupportedShape;
    if (!wsp || wsb < kHead || !aligned16(wsp)) return kErrWorkspace;
    auto st = static_cast<cudaStream_t>(stream);
    auto* ws = static_cast<ScalarsWs*>(wsp);
    int rc = launch_zero_scalars(ws, st);
    if (rc) return rc;
    rc = launch_amax_nnz_flat(in, dtype == MOR_B200_FP32, n, ws, st);
    if (rc) return rc;
    export_scalars_kernel<<<1, 1, 0, st>>>(ws, amax_out, reinterpret_cast<long long*>(nnz_out));
    return check_launch();
}

}  // extern "C"
