// Thin PyTorch front end over the C ABI of libmor_b200 (include/mor_b200.h).
//
// Registers the operator schemas of the reference extension verbatim
// (mor/csrc/fake_quantize.cpp:12-25 of boryiings/mor) under torch.ops.mor.*, for the
// CUDA dispatch key only -- there is no CPU implementation and none is wanted.  The
// shim validates arguments with TORCH_CHECK, allocates outputs and the workspace with
// torch::empty on the input's device, and launches on the CURRENT stream (the
// reference uses the legacy default stream).  It holds no arithmetic.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "../../include/mor_b200.h"

namespace mor {

namespace {

void* cur_stream() { return static_cast<void*>(at::cuda::getCurrentCUDAStream().stream()); }

void check_status(int rc, const char* op) {
    TORCH_CHECK(rc == MOR_B200_OK, "mor::", op, ": ", mor_b200_status_string(rc), " (status ", rc, ")");
}

int dtype_code(const at::Tensor& t, bool allow_fp32, const char* op) {
    if (t.dtype() == at::kBFloat16) return MOR_B200_BF16;
    TORCH_CHECK(allow_fp32 && t.dtype() == at::kFloat, "mor::", op, ": input must be bfloat16",
                allow_fp32 ? " or float32" : "");
    return MOR_B200_FP32;
}

at::Tensor checked_input(const at::Tensor& input, int64_t rows, int64_t cols, const char* op) {
    TORCH_CHECK(input.is_cuda(), "mor::", op, ": input must be a CUDA tensor");
    TORCH_CHECK(input.dim() == 2 && input.size(0) == rows && input.size(1) == cols, "mor::", op,
                ": input must be [dim_x, dim_y] = [", rows, ", ", cols, "]");
    return input.contiguous();
}

at::Tensor workspace(const at::Tensor& like, size_t bytes) {
    return torch::empty({(int64_t)bytes}, like.options().dtype(torch::kUInt8));
}

at::Tensor meta_tensor(const at::Tensor& like, int64_t rows, int64_t cols, int64_t br, int64_t bc) {
    const int64_t gx = (cols / 2 - 1) / (bc / 2) + 1, gy = (rows - 1) / br + 1;  // fake_quantize.cu:1757-1761
    return torch::empty({gy, gx}, like.options().dtype(torch::kInt32));
}

void check_fq_args(int64_t rows, int64_t cols, int64_t br, int64_t bc, int64_t sf_type) {
    TORCH_CHECK(rows > 0 && cols > 0 && br > 0 && bc >= 2, "mor::fake_quantize: sizes must be positive");
    TORCH_CHECK(cols % 2 == 0 && bc % 2 == 0, "mor::fake_quantize: dim_y and block_y must be even");
    TORCH_CHECK(sf_type == 1 || sf_type == 2, "mor::fake_quantize: sf_type must be 1 (fp32) or 2 (e8)");
}

// ---- fake_quantize ---------------------------------------------------------------
std::vector<at::Tensor> fake_quantize(const at::Tensor& input, int64_t rows, int64_t cols, int64_t br, int64_t bc,
                                      double clamp, int64_t mode, int64_t sf_type) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, "fake_quantize");
    const int dt = dtype_code(in, true, "fake_quantize");
    check_fq_args(rows, cols, br, bc, sf_type);
    at::Tensor out = torch::empty_like(in);
    at::Tensor meta = meta_tensor(in, rows, cols, br, bc);
    check_status(mor_b200_fake_quantize(in.data_ptr(), out.data_ptr(), meta.data_ptr<int32_t>(), dt, rows, cols,
                                        (int)br, (int)bc, clamp, (int)mode, (int)sf_type, cur_stream()),
                 "fake_quantize");
    return {out, meta};
}

at::Tensor fake_quantize_no_alloc(const at::Tensor& input, int64_t rows, int64_t cols, int64_t br, int64_t bc,
                                  double clamp, int64_t mode, int64_t sf_type, at::Tensor& result) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, "fake_quantize_no_alloc");
    const int dt = dtype_code(in, true, "fake_quantize_no_alloc");
    check_fq_args(rows, cols, br, bc, sf_type);
    TORCH_CHECK(result.is_cuda() && result.dtype() == in.dtype() && result.is_contiguous() && result.dim() == 2 &&
                    result.size(0) == rows && result.size(1) == cols,
                "mor::fake_quantize_no_alloc: result must be a contiguous CUDA tensor shaped and typed like input");
    at::Tensor meta = meta_tensor(in, rows, cols, br, bc);
    check_status(mor_b200_fake_quantize(in.data_ptr(), result.data_ptr(), meta.data_ptr<int32_t>(), dt, rows, cols,
                                        (int)br, (int)bc, clamp, (int)mode, (int)sf_type, cur_stream()),
                 "fake_quantize_no_alloc");
    return meta;
}

// ---- test operators ----------------------------------------------------------------
at::Tensor quant_dequant(const at::Tensor& input, int64_t rows, int64_t cols, int format, const char* op) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, op);
    TORCH_CHECK(in.dtype() == at::kFloat, "mor::", op, ": input must be float32");
    at::Tensor out = torch::empty_like(in);
    check_status(mor_b200_quant_dequant(in.data_ptr<float>(), out.data_ptr<float>(), rows, cols, format, cur_stream()), op);
    return out;
}
at::Tensor quant_dequant_e4m3(const at::Tensor& t, int64_t r, int64_t c, int64_t, int64_t) { return quant_dequant(t, r, c, MOR_B200_E4M3, "quant_dequant_e4m3"); }
at::Tensor quant_dequant_e5m2(const at::Tensor& t, int64_t r, int64_t c, int64_t, int64_t) { return quant_dequant(t, r, c, MOR_B200_E5M2, "quant_dequant_e5m2"); }
at::Tensor quant_dequant_e3m2(const at::Tensor& t, int64_t r, int64_t c, int64_t, int64_t) { return quant_dequant(t, r, c, MOR_B200_E3M2, "quant_dequant_e3m2"); }
at::Tensor quant_dequant_e2m3(const at::Tensor& t, int64_t r, int64_t c, int64_t, int64_t) { return quant_dequant(t, r, c, MOR_B200_E2M3, "quant_dequant_e2m3"); }

at::Tensor e8_scale(const at::Tensor& input, int64_t rows, int64_t cols, int rne, const char* op) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, op);
    TORCH_CHECK(in.dtype() == at::kFloat, "mor::", op, ": input must be float32");
    at::Tensor out = torch::empty_like(in);
    check_status(mor_b200_e4m3_with_e8_scale(in.data_ptr<float>(), out.data_ptr<float>(), rows, cols, rne, cur_stream()), op);
    return out;
}
at::Tensor e4m3_with_e8_scale_rne(const at::Tensor& t, int64_t r, int64_t c, int64_t, int64_t) { return e8_scale(t, r, c, 1, "e4m3_with_e8_scale_rne"); }
at::Tensor e4m3_with_e8_scale_rz(const at::Tensor& t, int64_t r, int64_t c, int64_t, int64_t) { return e8_scale(t, r, c, 0, "e4m3_with_e8_scale_rz"); }

// ---- block / channel scaling ---------------------------------------------------------
// Returns [out, meta, global_amax, global_non_zero, global_error]; inplace drops `out`.
// bf16 inputs report the non-zero count as int32 like the reference; float32 inputs
// (an extension for tensors of 2^31 elements and more) report int64.
std::vector<at::Tensor> scaling(int op, const char* name, at::Tensor in, at::Tensor out, int64_t rows, int64_t cols,
                                int64_t br, int64_t bc, double thr, int64_t ss) {
    const int dt = dtype_code(in, true, name);
    TORCH_CHECK(ss >= 1 && ss <= 4, "mor::", name, ": ss_mode must be 1..4");
    TORCH_CHECK(br > 0 && bc > 0 && rows % br == 0 && cols % bc == 0, "mor::", name,
                ": block shape must divide the tensor");
    if (op == MOR_B200_OP_CHANNEL_SCALING)
        TORCH_CHECK(br == 1 || bc == 1, "mor::", name, ": block_x or block_y must be 1");
    TORCH_CHECK(dt == MOR_B200_FP32 || rows * cols < (int64_t(1) << 31), "mor::", name,
                ": bfloat16 tensors report an int32 non-zero count; use float32 for 2^31 elements and more");
    const size_t wsb = mor_b200_workspace_bytes(op, rows, cols, (int)br, (int)bc);
    TORCH_CHECK(wsb > 0, "mor::", name, ": unsupported block shape ", br, " x ", bc);
    at::Tensor ws = workspace(in, wsb);
    auto iopt = in.options().dtype(torch::kInt32);
    auto fopt = in.options().dtype(torch::kFloat);
    at::Tensor meta = torch::empty({1}, iopt), gamax = torch::empty({1}, fopt), gerr = torch::empty({1}, fopt);
    const bool nnz64 = dt == MOR_B200_FP32;
    at::Tensor gnnz = torch::empty({1}, nnz64 ? in.options().dtype(torch::kInt64) : iopt);
    auto fn = op == MOR_B200_OP_BLOCK_SCALING ? mor_b200_block_scaling : mor_b200_channel_scaling;
    check_status(fn(in.data_ptr(), out.data_ptr(), dt, rows, cols, (int)br, (int)bc, thr, (int)ss,
                    meta.data_ptr<int32_t>(), gamax.data_ptr<float>(), gnnz.data_ptr(), nnz64 ? 1 : 0,
                    gerr.data_ptr<float>(), ws.data_ptr(), wsb, cur_stream()),
                 name);
    return {out, meta, gamax, gnnz, gerr};
}

std::vector<at::Tensor> fake_quantize_block_scaling(const at::Tensor& input, int64_t rows, int64_t cols, int64_t br,
                                                    int64_t bc, double thr, int64_t ss) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, "fake_quantize_block_scaling");
    return scaling(MOR_B200_OP_BLOCK_SCALING, "fake_quantize_block_scaling", in, torch::empty_like(in), rows, cols, br, bc, thr, ss);
}
std::vector<at::Tensor> fake_quantize_channel_scaling(const at::Tensor& input, int64_t rows, int64_t cols, int64_t br,
                                                      int64_t bc, double thr, int64_t ss) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, "fake_quantize_channel_scaling");
    return scaling(MOR_B200_OP_CHANNEL_SCALING, "fake_quantize_channel_scaling", in, torch::empty_like(in), rows, cols, br, bc, thr, ss);
}
std::vector<at::Tensor> scaling_inplace(int op, const char* name, at::Tensor& input, int64_t rows, int64_t cols,
                                        int64_t br, int64_t bc, double thr, int64_t ss) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, name);
    auto r = scaling(op, name, in, in, rows, cols, br, bc, thr, ss);
    if (!in.is_same(input)) input.copy_(in);  // a strided input was packed first
    return {r[1], r[2], r[3], r[4]};
}
std::vector<at::Tensor> fake_quantize_block_scaling_inplace(at::Tensor& input, int64_t rows, int64_t cols, int64_t br,
                                                            int64_t bc, double thr, int64_t ss) {
    return scaling_inplace(MOR_B200_OP_BLOCK_SCALING, "fake_quantize_block_scaling_inplace", input, rows, cols, br, bc, thr, ss);
}
std::vector<at::Tensor> fake_quantize_channel_scaling_inplace(at::Tensor& input, int64_t rows, int64_t cols,
                                                              int64_t br, int64_t bc, double thr, int64_t ss) {
    return scaling_inplace(MOR_B200_OP_CHANNEL_SCALING, "fake_quantize_channel_scaling_inplace", input, rows, cols, br, bc, thr, ss);
}

// ---- E8Mx -----------------------------------------------------------------------------
void e8mx_into(const at::Tensor& in, at::Tensor& out, int64_t rows, int64_t cols, int64_t qt, int64_t strat,
               const char* name) {
    TORCH_CHECK(in.dtype() == at::kBFloat16, "mor::", name, ": input must be bfloat16");
    TORCH_CHECK(qt >= 1 && qt <= 3, "mor::", name, ": quantize_type must be 1, 2 or 3");
    TORCH_CHECK(cols % 2 == 0, "mor::", name, ": dim_y must be even");
    const size_t wsb = mor_b200_workspace_bytes(MOR_B200_OP_E8MX, rows, cols, 0, 0);
    at::Tensor ws = workspace(in, wsb);
    check_status(mor_b200_e8mx(in.data_ptr(), out.data_ptr(), rows, cols, (int)qt, (int)strat, ws.data_ptr(), wsb,
                               cur_stream()),
                 name);
}
at::Tensor fake_quantize_e8mx(const at::Tensor& input, int64_t rows, int64_t cols, int64_t, int64_t, int64_t qt,
                              int64_t strat) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, "fake_quantize_e8mx");
    at::Tensor out = torch::empty_like(in);
    e8mx_into(in, out, rows, cols, qt, strat, "fake_quantize_e8mx");
    return out;
}
void fake_quantize_e8mx_inplace(const at::Tensor& input, int64_t rows, int64_t cols, int64_t, int64_t, int64_t qt,
                                int64_t strat, at::Tensor& result) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, "fake_quantize_e8mx_inplace");
    TORCH_CHECK(result.is_cuda() && result.dtype() == at::kBFloat16 && result.is_contiguous() && result.dim() == 2 &&
                    result.size(0) == rows && result.size(1) == cols,
                "mor::fake_quantize_e8mx_inplace: result must be a contiguous bfloat16 CUDA tensor shaped like input");
    e8mx_into(in, result, rows, cols, qt, strat, "fake_quantize_e8mx_inplace");
}

// ---- extension: per-group (MX) fake-quantize -------------------------------------------
// returns [out, scales]; scales is float32 [dim_x, dim_y / block_y]
std::vector<at::Tensor> fake_quantize_mx(const at::Tensor& input, int64_t rows, int64_t cols, int64_t bc,
                                         int64_t elem_format, int64_t sf_type) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, "fake_quantize_mx");
    const int dt = dtype_code(in, true, "fake_quantize_mx");
    TORCH_CHECK(bc > 0 && cols % bc == 0, "mor::fake_quantize_mx: block_y must divide dim_y");
    TORCH_CHECK(elem_format == MOR_B200_E4M3 || elem_format == MOR_B200_E5M2 || elem_format == MOR_B200_E2M3,
                "mor::fake_quantize_mx: elem_format must be 0 (E4M3), 1 (E5M2) or 3 (E2M3)");
    TORCH_CHECK(sf_type == 1 || sf_type == 2, "mor::fake_quantize_mx: sf_type must be 1 (fp32) or 2 (e8)");
    at::Tensor out = torch::empty_like(in);
    at::Tensor scales = torch::empty({rows, cols / bc}, in.options().dtype(torch::kFloat));
    check_status(mor_b200_fake_quantize_group(in.data_ptr(), out.data_ptr(), scales.data_ptr<float>(), dt, rows, cols,
                                              (int)bc, (int)elem_format, (int)sf_type, cur_stream()),
                 "fake_quantize_mx");
    return {out, scales};
}

// ---- extension: single-pass block scaling with a delayed tensor amax ---------------------
// returns [out, meta, amax of this tensor, non-zero count, error]; amax_in: float32[1] on the device
std::vector<at::Tensor> fake_quantize_block_scaling_delayed(const at::Tensor& input, int64_t rows, int64_t cols,
                                                            int64_t br, int64_t bc, double thr, int64_t ss,
                                                            const at::Tensor& amax_in) {
    const char* name = "fake_quantize_block_scaling_delayed";
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, name);
    const int dt = dtype_code(in, true, name);
    TORCH_CHECK(ss >= 1 && ss <= 4, "mor::", name, ": ss_mode must be 1..4");
    TORCH_CHECK(br == 128 && bc == 128 && rows % 128 == 0 && cols % 128 == 0, "mor::", name,
                ": 128 x 128 blocks that divide the tensor only");
    TORCH_CHECK(amax_in.is_cuda() && amax_in.scalar_type() == at::kFloat && amax_in.numel() == 1, "mor::", name,
                ": amax_in must be a float32 CUDA tensor with one element");
    TORCH_CHECK(dt == MOR_B200_FP32 || rows * cols < (int64_t(1) << 31), "mor::", name,
                ": bfloat16 tensors report an int32 non-zero count; use float32 for 2^31 elements and more");
    const size_t wsb = mor_b200_workspace_bytes(MOR_B200_OP_BLOCK_SCALING, rows, cols, 128, 128);
    at::Tensor ws = workspace(in, wsb);
    at::Tensor out = torch::empty_like(in);
    auto iopt = in.options().dtype(torch::kInt32);
    auto fopt = in.options().dtype(torch::kFloat);
    at::Tensor meta = torch::empty({1}, iopt), gamax = torch::empty({1}, fopt), gerr = torch::empty({1}, fopt);
    const bool nnz64 = dt == MOR_B200_FP32;
    at::Tensor gnnz = torch::empty({1}, nnz64 ? in.options().dtype(torch::kInt64) : iopt);
    check_status(mor_b200_block_scaling_delayed(in.data_ptr(), out.data_ptr(), dt, rows, cols, 128, 128, thr, (int)ss,
                                                amax_in.data_ptr<float>(), meta.data_ptr<int32_t>(),
                                                gamax.data_ptr<float>(), gnnz.data_ptr(), nnz64 ? 1 : 0,
                                                gerr.data_ptr<float>(), ws.data_ptr(), wsb, cur_stream()),
                 name);
    return {out, meta, gamax, gnnz, gerr};
}

// the same, and the result transposed as well: returns [out, out_t [dim_y, dim_x], meta, amax, non-zero count, error]
std::vector<at::Tensor> fake_quantize_block_scaling_delayed_t(const at::Tensor& input, int64_t rows, int64_t cols,
                                                              int64_t br, int64_t bc, double thr, int64_t ss,
                                                              const at::Tensor& amax_in) {
    const char* name = "fake_quantize_block_scaling_delayed_t";
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, name);
    const int dt = dtype_code(in, true, name);
    TORCH_CHECK(ss >= 1 && ss <= 4, "mor::", name, ": ss_mode must be 1..4");
    TORCH_CHECK(br == 128 && bc == 128 && rows % 128 == 0 && cols % 128 == 0, "mor::", name,
                ": 128 x 128 blocks that divide the tensor only");
    TORCH_CHECK(amax_in.is_cuda() && amax_in.scalar_type() == at::kFloat && amax_in.numel() == 1, "mor::", name,
                ": amax_in must be a float32 CUDA tensor with one element");
    TORCH_CHECK(dt == MOR_B200_FP32 || rows * cols < (int64_t(1) << 31), "mor::", name,
                ": bfloat16 tensors report an int32 non-zero count; use float32 for 2^31 elements and more");
    const size_t wsb = mor_b200_workspace_bytes(MOR_B200_OP_BLOCK_SCALING, rows, cols, 128, 128);
    at::Tensor ws = workspace(in, wsb);
    at::Tensor out = torch::empty_like(in);
    at::Tensor out_t = torch::empty({cols, rows}, in.options());
    auto iopt = in.options().dtype(torch::kInt32);
    auto fopt = in.options().dtype(torch::kFloat);
    at::Tensor meta = torch::empty({1}, iopt), gamax = torch::empty({1}, fopt), gerr = torch::empty({1}, fopt);
    const bool nnz64 = dt == MOR_B200_FP32;
    at::Tensor gnnz = torch::empty({1}, nnz64 ? in.options().dtype(torch::kInt64) : iopt);
    check_status(mor_b200_block_scaling_delayed_t(in.data_ptr(), out.data_ptr(), out_t.data_ptr(), dt, rows, cols, 128, 128,
                                                  thr, (int)ss, amax_in.data_ptr<float>(), meta.data_ptr<int32_t>(),
                                                  gamax.data_ptr<float>(), gnnz.data_ptr(), nnz64 ? 1 : 0,
                                                  gerr.data_ptr<float>(), ws.data_ptr(), wsb, cur_stream()),
                 name);
    return {out, out_t, meta, gamax, gnnz, gerr};
}

// ---- extension: real quantized output (codes + E8M0 scale bytes) -----------------------
// returns [payload uint8 [dim_x, dim_y], scales uint8 [dim_x, dim_y / block_y]]
std::vector<at::Tensor> quantize_mx(const at::Tensor& input, int64_t rows, int64_t cols, int64_t bc, int64_t elem_format) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, "quantize_mx");
    TORCH_CHECK(in.scalar_type() == at::kBFloat16, "mor::quantize_mx: bfloat16 input only");
    TORCH_CHECK(bc > 0 && cols % bc == 0, "mor::quantize_mx: block_y must divide dim_y");
    TORCH_CHECK(elem_format == MOR_B200_E4M3 || elem_format == MOR_B200_E5M2 || elem_format == MOR_B200_E2M3,
                "mor::quantize_mx: elem_format must be 0 (E4M3), 1 (E5M2) or 3 (E2M3)");
    at::Tensor payload = torch::empty({rows, cols}, in.options().dtype(torch::kUInt8));
    at::Tensor scales = torch::empty({rows, cols / bc}, in.options().dtype(torch::kUInt8));
    check_status(mor_b200_quantize_mx(in.data_ptr(), payload.data_ptr(), scales.data_ptr(), rows, cols, (int)bc,
                                      (int)elem_format, cur_stream()),
                 "quantize_mx");
    return {payload, scales};
}

// returns [payload uint8 [dim_x, dim_y * 3 / 4] (E2M3, six bits per element), scales uint8 [dim_x, dim_y / block_y]]
std::vector<at::Tensor> quantize_mx_fp6(const at::Tensor& input, int64_t rows, int64_t cols, int64_t bc) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, "quantize_mx_fp6");
    TORCH_CHECK(in.scalar_type() == at::kBFloat16, "mor::quantize_mx_fp6: bfloat16 input only");
    TORCH_CHECK(bc > 0 && cols % bc == 0 && cols % 8 == 0, "mor::quantize_mx_fp6: block_y must divide dim_y, dim_y a multiple of 8");
    at::Tensor payload = torch::empty({rows, cols * 3 / 4}, in.options().dtype(torch::kUInt8));
    at::Tensor scales = torch::empty({rows, cols / bc}, in.options().dtype(torch::kUInt8));
    check_status(mor_b200_quantize_mx_fp6(in.data_ptr(), payload.data_ptr(), scales.data_ptr(), rows, cols, (int)bc,
                                          cur_stream()),
                 "quantize_mx_fp6");
    return {payload, scales};
}

// returns [payload uint8 [dim_x, dim_y] (E4M3 bytes), scales float32 [dim_x / block_x, dim_y / block_y], global_amax float32[1]]
std::vector<at::Tensor> quantize_scaled(const at::Tensor& input, int64_t rows, int64_t cols, int64_t br, int64_t bc,
                                        int64_t ss) {
    const c10::cuda::CUDAGuard guard(input.device());
    at::Tensor in = checked_input(input, rows, cols, "quantize_scaled");
    const int dt = dtype_code(in, true, "quantize_scaled");
    TORCH_CHECK(ss == 1 || ss == 3 || ss == 4, "mor::quantize_scaled: ss_mode must be 1, 3 or 4 (binary32 scales)");
    TORCH_CHECK(br > 0 && bc > 0 && rows % br == 0 && cols % bc == 0, "mor::quantize_scaled: block shape must divide the tensor");
    const int op = (br == 1 || bc == 1) ? MOR_B200_OP_CHANNEL_SCALING : MOR_B200_OP_BLOCK_SCALING;
    const size_t wsb = mor_b200_workspace_bytes(op, rows, cols, (int)br, (int)bc);
    TORCH_CHECK(wsb > 0, "mor::quantize_scaled: unsupported block shape ", br, " x ", bc);
    at::Tensor ws = workspace(in, wsb);
    at::Tensor payload = torch::empty({rows, cols}, in.options().dtype(torch::kUInt8));
    at::Tensor scales = torch::empty({rows / br, cols / bc}, in.options().dtype(torch::kFloat));
    at::Tensor gamax = torch::empty({1}, in.options().dtype(torch::kFloat));
    check_status(mor_b200_quantize_scaled(in.data_ptr(), payload.data_ptr(), scales.data_ptr<float>(), dt, rows, cols, (int)br,
                                          (int)bc, (int)ss, nullptr, gamax.data_ptr<float>(), ws.data_ptr(), wsb, cur_stream()),
                 "quantize_scaled");
    return {payload, scales, gamax};
}

}  // namespace

// Registers _C as a Python extension module.
PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {}

TORCH_LIBRARY(mor, m) {
  // the fourteen schemas of the reference, unchanged
  m.def("fake_quantize(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float clamp_threshold, int mode, int sf_type) -> Tensor[]");
  m.def("fake_quantize_no_alloc(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float clamp_threshold, int mode, int sf_type, Tensor result) -> Tensor");
  m.def("quant_dequant_e4m3(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor");
  m.def("quant_dequant_e5m2(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor");
  m.def("quant_dequant_e3m2(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor");
  m.def("quant_dequant_e2m3(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor");
  m.def("e4m3_with_e8_scale_rne(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor");
  m.def("e4m3_with_e8_scale_rz(Tensor input, int dim_x, int dim_y, int block_x, int block_y) -> Tensor");
  m.def("fake_quantize_block_scaling(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float e4m3_threshold, int ss_mode) -> Tensor[]");
  m.def("fake_quantize_block_scaling_inplace(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float e4m3_threshold, int ss_mode) -> Tensor[]");
  m.def("fake_quantize_e8mx(Tensor input, int dim_x, int dim_y, int block_x, int block_y, int quantize_type, int scaling_strategy) -> Tensor");
  m.def("fake_quantize_e8mx_inplace(Tensor input, int dim_x, int dim_y, int block_x, int block_y, int quantize_type, int scaling_strategy, Tensor result) -> ()");
  m.def("fake_quantize_channel_scaling(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float e4m3_threshold, int ss_mode) -> Tensor[]");
  m.def("fake_quantize_channel_scaling_inplace(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float e4m3_threshold, int ss_mode) -> Tensor[]");
  // addition: one scale per 1 x block_y group (MX), E4M3 / E5M2 / E2M3 elements
  m.def("fake_quantize_mx(Tensor input, int dim_x, int dim_y, int block_y, int elem_format, int sf_type) -> Tensor[]");
  m.def("quantize_mx(Tensor input, int dim_x, int dim_y, int block_y, int elem_format) -> Tensor[]");
  m.def("quantize_mx_fp6(Tensor input, int dim_x, int dim_y, int block_y) -> Tensor[]");
  m.def("quantize_scaled(Tensor input, int dim_x, int dim_y, int block_x, int block_y, int ss_mode) -> Tensor[]");
  m.def("fake_quantize_block_scaling_delayed(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float e4m3_threshold, int ss_mode, Tensor amax_in) -> Tensor[]");
  m.def("fake_quantize_block_scaling_delayed_t(Tensor input, int dim_x, int dim_y, int block_x, int block_y, float e4m3_threshold, int ss_mode, Tensor amax_in) -> Tensor[]");
}

TORCH_LIBRARY_IMPL(mor, CUDA, m) {
  m.impl("fake_quantize", &fake_quantize);
  m.impl("fake_quantize_no_alloc", &fake_quantize_no_alloc);
  m.impl("quant_dequant_e4m3", &quant_dequant_e4m3);
  m.impl("quant_dequant_e5m2", &quant_dequant_e5m2);
  m.impl("quant_dequant_e3m2", &quant_dequant_e3m2);
  m.impl("quant_dequant_e2m3", &quant_dequant_e2m3);
  m.impl("e4m3_with_e8_scale_rne", &e4m3_with_e8_scale_rne);
  m.impl("e4m3_with_e8_scale_rz", &e4m3_with_e8_scale_rz);
  m.impl("fake_quantize_block_scaling", &fake_quantize_block_scaling);
  m.impl("fake_quantize_block_scaling_inplace", &fake_quantize_block_scaling_inplace);
  m.impl("fake_quantize_e8mx", &fake_quantize_e8mx);
  m.impl("fake_quantize_e8mx_inplace", &fake_quantize_e8mx_inplace);
  m.impl("fake_quantize_channel_scaling", &fake_quantize_channel_scaling);
  m.impl("fake_quantize_channel_scaling_inplace", &fake_quantize_channel_scaling_inplace);
  m.impl("fake_quantize_mx", &fake_quantize_mx);
  m.impl("quantize_mx", &quantize_mx);
  m.impl("quantize_mx_fp6", &quantize_mx_fp6);
  m.impl("quantize_scaled", &quantize_scaled);
  m.impl("fake_quantize_block_scaling_delayed", &fake_quantize_block_scaling_delayed);
  m.impl("fake_quantize_block_scaling_delayed_t", &fake_quantize_block_scaling_delayed_t);
}

}  // namespace mor
