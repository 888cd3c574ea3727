/*
 * mor_b200 -- C ABI of the B200 (sm_100a) fake-quantization library.
 *
 * Every entry point takes raw DEVICE pointers, plain sizes and a CUDA stream
 * (cudaStream_t passed as void*), enqueues its kernels on that stream and returns
 * without synchronising.  Nothing here allocates: the operators that need scratch
 * memory take a caller-owned workspace whose size mor_b200_workspace_bytes()
 * reports.  The return value is a status code; no entry point throws or traps.
 *
 * Tensors are contiguous row-major [rows, cols], 16-byte aligned at the base.
 * dtype MOR_B200_BF16: bf16 in, bf16 out (the reference's only data type).
 * dtype MOR_B200_FP32: binary32 in, binary32 out with the same arithmetic minus the
 * bf16 widening/rounding steps (an extension; the reference has no such path).
 *
 * Each declaration cites the interface of the reference (boryiings/mor) that it
 * replaces: the operator schema in mor/csrc/fake_quantize.cpp and the host launcher
 * in mor/csrc/cuda/fake_quantize.cu.
 */
#ifndef MOR_B200_H_
#define MOR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* every entry point below is exported from libmor_b200.so; nothing else is */
#if defined(__GNUC__)
#define MOR_B200_API __attribute__((visibility("default")))
#else
#define MOR_B200_API
#endif

#define MOR_B200_OK 0
#define MOR_B200_ERR_INVALID_ARGUMENT (-1) /* bad pointer, size, mode or dtype               */
#define MOR_B200_ERR_UNSUPPORTED_SHAPE (-2) /* shape/alignment the kernels do not cover       */
#define MOR_B200_ERR_WORKSPACE (-3)        /* workspace missing or too small                 */
#define MOR_B200_ERR_LAUNCH (-4)           /* the CUDA runtime refused a launch              */
#define MOR_B200_ERR_TOO_LARGE (-5)        /* more blocks than a grid can index              */
#define MOR_B200_ERR_STATIC_SCRATCH (-6)   /* more blocks than the built-in scratch holds    */

#define MOR_B200_BF16 0
#define MOR_B200_FP32 1

/* narrow formats (quant_dequant, fake_quantize_group) */
#define MOR_B200_E4M3 0
#define MOR_B200_E5M2 1
#define MOR_B200_E3M2 2
#define MOR_B200_E2M3 3

/* operators that need a workspace */
#define MOR_B200_OP_BLOCK_SCALING 1
#define MOR_B200_OP_CHANNEL_SCALING 2
#define MOR_B200_OP_E8MX 3
#define MOR_B200_OP_AMAX_NNZ 4

MOR_B200_API int mor_b200_version(void);
MOR_B200_API const char* mor_b200_status_string(int status);

/* Test switch, no counterpart in the reference.  Several kernels can serve the same operator and all
 * give the same bits; the parity tests use this mask to run each of them on the same input.
 * bit 0: operators that would take a TMA-staged 128 x 128 tile kernel or a single-pass group kernel
 *        take the generic kernel for any block shape instead;
 * bit 1: block scaling does not take the single-launch kernel that keeps a small tensor in shared
 *        memory between its two passes (it then runs as the sequence of launches used for large tensors).
 * Process-wide, 0 by default, not meant for production callers. */
MOR_B200_API void mor_b200_debug_kernel_selection(int mask);

/* Bytes of device workspace for one call of `op` on a [rows, cols] tensor with the
 * given block shape (0 for operators that need none).  Replaces the torch::empty
 * temporaries of the reference launchers (fake_quantize.cu:2070-2078, 2272-2277,
 * 2489-2497). */
MOR_B200_API size_t mor_b200_workspace_bytes(int op, int64_t rows, int64_t cols, int block_rows, int block_cols);

/* mor::fake_quantize / mor::fake_quantize_no_alloc
 * (fake_quantize.cpp:12-13; fake_quantize.cu:1763-1907, kernel 684-852).
 * mode % 10: 1 MoR, 2 block E4M3, 3 block E5M2, 4 current-scaling E4M3, 5 current-
 * scaling E5M2 (clamp_threshold is then the scale), anything else BF16 pass-through;
 * mode / 100 > 0 selects MoR's dynamic-range criterion instead of the relative-error
 * one.  sf_type 1: binary32 scale, 2: power-of-two (E8) scale.
 * meta: int32 [ceil(rows/block_rows), ceil((cols/2)/(block_cols/2))].
 * output may alias input. */
MOR_B200_API int mor_b200_fake_quantize(const void* input, void* output, int32_t* meta, int dtype, int64_t rows, int64_t cols,
                           int block_rows, int block_cols, double clamp_threshold, int mode, int sf_type,
                           void* stream);

/* mor::quant_dequant_e4m3 / _e5m2 / _e3m2 / _e2m3 (fake_quantize.cpp:14-17;
 * fake_quantize.cu:1909-1964, kernel 854-863): binary32 -> format -> binary32, no
 * scaling, the reference's own cast (NaN on E4M3/E5M2 overflow, clamp for E3M2/E2M3). */
MOR_B200_API int mor_b200_quant_dequant(const float* input, float* output, int64_t rows, int64_t cols, int format, void* stream);

/* mor::e4m3_with_e8_scale_rne / _rz (fake_quantize.cpp:18-19; fake_quantize.cu:1966-2011,
 * kernel 865-875): per-element power-of-two scale from 448/x. */
MOR_B200_API int mor_b200_e4m3_with_e8_scale(const float* input, float* output, int64_t rows, int64_t cols, int rne,
                                void* stream);

/* mor::fake_quantize_block_scaling[_inplace] (fake_quantize.cpp:20-21;
 * fake_quantize.cu:2013-2230, kernels 951-1241).  ss_mode 1 global-mantissa, 2 block
 * amax with power-of-two scale, 3 block amax with binary32 scale, 4 tensor scale
 * (2 and 3 are that way round in the reference, and here).  block_rows % 32 == 0,
 * block_cols % 64 == 0.  Scalar outputs are device pointers: meta (1 = E4M3 kept,
 * 3 = tensor left in BF16), global_amax, global_nnz (int32, or int64 when
 * nnz_is_int64), global_error.  output == input gives the _inplace operator. */
MOR_B200_API int mor_b200_block_scaling(const void* input, void* output, int dtype, int64_t rows, int64_t cols, int block_rows,
                           int block_cols, double e4m3_threshold, int ss_mode, int32_t* meta, float* global_amax,
                           void* global_nnz, int nnz_is_int64, float* global_error, void* workspace,
                           size_t workspace_bytes, void* stream);

/* mor_b200_block_scaling without a workspace argument.  No counterpart in the reference.
 *
 * For hosts that may not allocate device memory at the point of the call: code running
 * inside a CUDA-graph capture or another runtime's stream callback, plugins handed a
 * fixed set of buffers by their framework, services whose memory is carved up front by
 * an arena they do not own.  The scratch the pipeline needs (scalar head, one amax and
 * one error sum per block) lives in an array built into the library instead:
 * 4352 B + 8 B x 65536 blocks = 516.25 KiB of device memory on every GPU that loads the
 * library, held until the process exits.  Tensors with more than 65536 blocks (e.g. more
 * than 32768 x 32768 elements at 128 x 128) get MOR_B200_ERR_STATIC_SCRATCH; use
 * mor_b200_block_scaling for those.
 *
 * This call performs no cudaMalloc / cudaFree and calls no allocating library routine.
 * Its FIRST call on a device looks up the device address of the built-in array (once per
 * device, that device current); make that first call outside any stream capture.
 * All calls on a device share the one array: it keeps the previous call's contents (the
 * call clears or overwrites everything it later reads), and two calls whose kernels
 * overlap on the GPU -- different streams, or different host threads -- race on it.
 * Same arguments and results as mor_b200_block_scaling otherwise. */
MOR_B200_API int mor_b200_block_scaling_static(const void* input, void* output, int dtype, int64_t rows, int64_t cols,
                                  int block_rows, int block_cols, double e4m3_threshold, int ss_mode, int32_t* meta,
                                  float* global_amax, void* global_nnz, int nnz_is_int64, float* global_error,
                                  void* stream);

/* mor::fake_quantize_channel_scaling[_inplace] (fake_quantize.cpp:24-25;
 * fake_quantize.cu:2399-2660, kernels 1430-1752).  block_rows == 1 (1 x k row groups,
 * k a multiple of 128, or k in {8,16,32,64} with cols % 128 == 0) or block_cols == 1
 * (k x 1 column groups, k % 16 == 0, cols % 64 == 0).  Launch geometry is that of the
 * reference's e2m3 fork (e2m3/fake_quantize_e2m3.cu:2518), under which every group is
 * visited once. */
MOR_B200_API int mor_b200_channel_scaling(const void* input, void* output, int dtype, int64_t rows, int64_t cols, int block_rows,
                             int block_cols, double e4m3_threshold, int ss_mode, int32_t* meta, float* global_amax,
                             void* global_nnz, int nnz_is_int64, float* global_error, void* workspace,
                             size_t workspace_bytes, void* stream);

/* mor::fake_quantize_e8mx / _inplace (fake_quantize.cpp:22-23; fake_quantize.cu:2232-2397,
 * kernels 1243-1428).  quantize_type 1..3 = mantissa bits kept; scaling_strategy 1 =
 * scale by the tensor amax, anything else = unscaled.  bf16 only. */
MOR_B200_API int mor_b200_e8mx(const void* input, void* output, int64_t rows, int64_t cols, int quantize_type,
                  int scaling_strategy, void* workspace, size_t workspace_bytes, void* stream);

/* Extension (no reference operator; element semantics of quantize_kernel's
 * BLOCK_SCALING modes, fake_quantize.cu:801-823, with the SQDD wrappers :356-379):
 * single-pass fake-quantize with one scale per 1 x block_cols group, formats E4M3,
 * E5M2, E2M3, scale binary32 (sf_type 1) or power of two / E8M0 (sf_type 2).
 * scales (optional, device, one float per group) receives the scale applied. */
MOR_B200_API int mor_b200_fake_quantize_group(const void* input, void* output, float* scales, int dtype, int64_t rows,
                                 int64_t cols, int block_cols, int format, int sf_type, void* stream);

/* Extension (no counterpart in the reference; arithmetic of fake_quantize_block_scaling,
 * fake_quantize.cu:1059-1241, with the tensor amax supplied by the caller): block scaling in ONE
 * pass over the tensor.  The scales are built from *amax_in (device), typically the amax this
 * call reported for the previous step's tensor ("delayed scaling"); each block's own amax is
 * taken from the tile while it is staged on chip; amax_out / nnz_out / err_out / meta describe
 * THIS tensor.  128 x 128 blocks, input != output.  Values above the stale amax saturate in the
 * cast, as they do in the reference's arithmetic for a scale that is too large. */
MOR_B200_API int mor_b200_block_scaling_delayed(const void* input, void* output, int dtype, int64_t rows, int64_t cols,
                                   int block_rows, int block_cols, double e4m3_threshold, int ss_mode,
                                   const float* amax_in, int32_t* meta, float* amax_out, void* nnz_out,
                                   int nnz_is_int64, float* err_out, void* workspace, size_t workspace_bytes,
                                   void* stream);

/* mor_b200_block_scaling_delayed that also writes the result transposed: output_t is [cols, rows], the
 * layout a weight-gradient GEMM reads, produced from the tile while it is still on chip instead of by a
 * second pass over the tensor.  output may be NULL (transposed result only).  If the tensor stays BF16
 * (meta 3) output_t receives the transposed input.  No counterpart in the reference. */
MOR_B200_API int mor_b200_block_scaling_delayed_t(const void* input, void* output, void* output_t, int dtype, int64_t rows,
                                     int64_t cols, int block_rows, int block_cols, double e4m3_threshold, int ss_mode,
                                     const float* amax_in, int32_t* meta, float* amax_out, void* nnz_out,
                                     int nnz_is_int64, float* err_out, void* workspace, size_t workspace_bytes,
                                     void* stream);

/* Extension (no counterpart in the reference, whose operators only fake-quantize; the casts
 * it describes are fake_quantize.cu:283-305 and the wrappers :356-379): the REAL quantized form
 * of mor_b200_fake_quantize_group with sf_type 2, i.e. what a block-scaled GEMM consumes.
 * input: bf16 [rows, cols], 16-byte aligned.  payload: one byte per element [rows, cols], 8-byte
 * aligned -- the fp8 code for E4M3 (format 0) / E5M2 (1), the 6-bit code in a byte for E2M3 (3).
 * scales: one E8M0 byte per 1 x block_cols group [rows, cols / block_cols], MX convention:
 * element = decode(code) * 2^(scale - 127); an all-zero group gets 127.  block_cols a power of
 * two from 8 to 256, rows * cols a multiple of 256.  decode * scale equals the fake-quantized
 * output bit for bit, except where the code is zero under a scale below one (fake quantization
 * returns 2^(-e8-127) there, an artefact of its exponent-field arithmetic, :296-305). */
MOR_B200_API int mor_b200_quantize_mx(const void* input, void* payload, void* scales, int64_t rows, int64_t cols,
                         int block_cols, int format, void* stream);

/* The same with E2M3 elements packed six bits each: payload is [rows, cols * 3 / 4] bytes (2-byte
 * aligned), every run of eight elements a little-endian 48-bit group with code i in bits
 * [6 i, 6 i + 6).  No counterpart in the reference. */
MOR_B200_API int mor_b200_quantize_mx_fp6(const void* input, void* payload, void* scales, int64_t rows, int64_t cols,
                             int block_cols, void* stream);

/* Extension (no counterpart in the reference, whose operators only fake-quantize; the scale is
 * get_scaling_factor, fake_quantize.cu:1059-1093, the cast the one inside SQDD_fp32_scale, :310-316): the
 * REAL quantized form of mor_b200_block_scaling / mor_b200_channel_scaling under a binary32 scale
 * (ss_mode 1, 3 or 4).  payload: one E4M3 byte per element [rows, cols], 8-byte aligned, cols % 8 == 0;
 * scales: one float per block [rows / block_rows, cols / block_cols] (k x 1 blocks: one per column of
 * every row block).  element = decode(code) / scale -- the reference's division -- equals the
 * fake-quantized value bit for bit; a zero element gets code 0.  amax_in (device, optional): amax of the
 * whole tensor when `input` is a slab of it (row sharding), NULL to use this tensor's; amax_out
 * (device, optional) receives the amax used.  Block shapes as for the two operators, except 1 x k groups
 * of fewer than 128 columns.  Workspace: mor_b200_workspace_bytes of the matching operator. */
MOR_B200_API int mor_b200_quantize_scaled(const void* input, void* payload, float* scales, int dtype, int64_t rows,
                             int64_t cols, int block_rows, int block_cols, int ss_mode, const float* amax_in,
                             float* amax_out, void* workspace, size_t workspace_bytes, void* stream);

/* ---- row-sharded pipeline (extension): the phases of block/channel scaling as separate
 * calls, so that a caller holding one row slab per GPU can all-reduce the amax (max)
 * and the non-zero count (sum) and all-gather the block errors between them. ---- */

/* Phase 1 (kernels 951-1049 / 1459-1631): per-block amax into the workspace, slab amax
 * and non-zero count to amax_out / nnz_out (device; both may be NULL when the peer exchange
 * below takes them from the workspace). kind = MOR_B200_OP_BLOCK_SCALING or
 * MOR_B200_OP_CHANNEL_SCALING. */
MOR_B200_API int mor_b200_scaling_amax(int kind, const void* input, int dtype, int64_t rows, int64_t cols, int block_rows,
                          int block_cols, float* amax_out, int64_t* nnz_out, void* workspace, size_t workspace_bytes,
                          void* stream);
/* Phase 2 (kernels 1095-1176 / 1633-1752): scale, cast, store, per-CTA error sums.
 * global_amax: device pointer to the amax of the WHOLE tensor.  block_err_out: device
 * array of mor_b200_scaling_num_errors() floats.  Uses the block amax left in the
 * workspace by phase 1. */
MOR_B200_API int mor_b200_scaling_cast(int kind, const void* input, void* output, int dtype, int64_t rows, int64_t cols,
                          int block_rows, int block_cols, int ss_mode, const float* global_amax, float* block_err_out,
                          void* workspace, size_t workspace_bytes, void* stream);
MOR_B200_API int64_t mor_b200_scaling_num_errors(int kind, int64_t rows, int64_t cols, int block_rows, int block_cols);
/* slots of the reference's error array per stored sum (1, or blocks per CTA) */
MOR_B200_API int mor_b200_scaling_error_stride(int kind, int block_rows, int block_cols);
/* Phase 3 (kernels 1178-1241): ordered sum of ALL slabs' errors (concatenated in row
 * order), error / nnz against the threshold.  Writes meta (1 or 3) and global_error. */
MOR_B200_API int mor_b200_scaling_finalize(const float* block_err, int64_t n_err, int error_stride, const int64_t* global_nnz,
                              double e4m3_threshold, int32_t* meta, float* global_error, void* workspace,
                              size_t workspace_bytes, void* stream);
/* Phase 4: if *meta == 3, copy the slab's input over its output. */
MOR_B200_API int mor_b200_scaling_fallback(const void* input, void* output, int64_t n_bytes, const int32_t* meta, void* stream);

/* ---- peer exchange for the row-sharded pipeline (extension; the reference is single-GPU) ----
 * Replaces the scalar all-reduces and the all-gather of the error sums by plain NVLink stores
 * into a buffer that every rank allocates (mor_b200_p2p_alloc with mor_b200_p2p_bytes) and maps
 * from all its peers (mor_b200_p2p_open); peer_bufs[r] is rank r's buffer as seen from this process
 * (peer_bufs[rank] = the own one).  epoch counts the calls (1, 2, ...; the same on every rank).
 * Order per call, all on one stream:  scaling_amax (its two outputs may be NULL) ->
 * p2p_exchange_scalars (writes global amax and nnz) -> scaling_cast -> p2p_exchange_errors ->
 * scaling_finalize on (own buffer + p2p_error_offset, world * n_err entries) -> scaling_fallback.
 * Waits are bounded (several seconds); a time-out sets a flag in the workspace head and
 * scaling_finalize then reports meta = -1.  world <= 16. */
/* The exchange buffer is allocated (cudaMalloc, zero-filled), exported (64-byte CUDA IPC handle,
 * to be sent to the other processes by any means) and opened by the library: a peer's buffer must
 * be opened while `device`, the GPU whose kernels will store into it, is current.  close() unmaps
 * a peer's buffer, free() releases the own one (after every peer has closed it). */
#define MOR_B200_P2P_HANDLE_BYTES 64
MOR_B200_API int mor_b200_p2p_alloc(int device, size_t bytes, void** ptr_out, unsigned char* handle_out);
MOR_B200_API int mor_b200_p2p_open(int device, const unsigned char* handle, void** ptr_out);
MOR_B200_API int mor_b200_p2p_close(int device, void* peer_ptr);
MOR_B200_API int mor_b200_p2p_free(int device, void* own_ptr);
MOR_B200_API size_t mor_b200_p2p_bytes(int world, int64_t n_err);
/* polls (about 0.3 us each) after which a wait of the exchange kernels gives up; default 2^25 */
MOR_B200_API void mor_b200_p2p_set_wait_limit(uint32_t polls);
MOR_B200_API size_t mor_b200_p2p_error_offset(int world, int64_t n_err, uint32_t epoch);
MOR_B200_API int mor_b200_p2p_exchange_scalars(void* workspace, void* my_buf, void* const* peer_bufs, int rank, int world,
                                  uint32_t epoch, float* global_amax, int64_t* global_nnz, void* stream);
/* Phase 1 and the exchange of its scalars in one kernel (no reference counterpart): as mor_b200_scaling_amax,
 * and the CTA that finishes last stores the slab's amax and count into every peer's buffer, flags, waits
 * (bounded) for the peers' and writes the tensor's amax and count to global_amax / global_nnz -- what
 * mor_b200_p2p_exchange_scalars does in a launch of its own.  MOR_B200_ERR_UNSUPPORTED_SHAPE, with nothing
 * launched, for block shapes whose amax kernel has no built-in exchange (k x 1 and long 1 x k groups, flat
 * tensors): call the two separately then. */
MOR_B200_API int mor_b200_scaling_amax_p2p(int kind, const void* input, int dtype, int64_t rows, int64_t cols,
                              int block_rows, int block_cols, void* workspace, size_t workspace_bytes, void* my_buf,
                              void* const* peer_bufs, int rank, int world, uint32_t epoch, float* global_amax,
                              int64_t* global_nnz, void* stream);
MOR_B200_API int mor_b200_p2p_exchange_errors(const float* local_err, int64_t n_err, const void* my_buf,
                                 void* const* peer_bufs, int rank, int world, uint32_t epoch, void* workspace,
                                 void* stream);

/* amax and non-zero count of a flat tensor (kernels 951-1049 without the block array). */
MOR_B200_API int mor_b200_amax_nnz(const void* input, int dtype, int64_t n_elems, float* amax_out, int64_t* nnz_out,
                      void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOR_B200_H_ */
