/*
 * C ABI of libcomfy_kitchen_b200.so — the sm_100a kernels of comfy-kitchen's
 * quantized-linear hot path (FP8 / NVFP4 / MXFP8 quantizers, block-scaled GEMMs,
 * RoPE, AdaLN and the fused AdaLN->quantize front end).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer on the current device unless stated;
 *     the library never allocates, frees or synchronises (the two
 *     ck_*_device_status calls excepted, which synchronise) and launches on the stream it is given;
 *   - dtype codes: 0 float32, 1 float16, 2 bfloat16, 5 float8_e4m3fn, 6 float8_e5m2
 *     (comfy_kitchen/backends/eager/quantization.py:33-41);
 *   - block scales use the 128x4 tiled layout of
 *     comfy_kitchen/float_utils.py:292-326 (to_blocked): scale (r, c) of a tensor
 *     with C scale columns (C rounded up to 4) lives at byte
 *       ((r/128)*(C/4) + c/4)*512 + (r%32)*16 + ((r%128)/32)*4 + c%4
 *     and the buffer covers rows rounded up to 128; quantizers write every byte
 *     of it (padding = 0);
 *   - return value: 0 success; negative = argument error (CK_ERR_*); positive =
 *     cudaError_t of the launch.  ck_last_error() returns a description for the
 *     calling thread.  The reference's entry points of the same names
 *     (comfy_kitchen/backends/cuda/dlpack_bindings.cpp:44-209) return void and
 *     throw C++ exceptions; everything else about their signatures is kept.
 */
#ifndef COMFY_KITCHEN_B200_H_
#define COMFY_KITCHEN_B200_H_

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* ck_stream_t; /* cudaStream_t */

#define CK_OK 0
#define CK_ERR_DTYPE (-1)
#define CK_ERR_SHAPE (-2)
#define CK_ERR_ALIGN (-3)
#define CK_ERR_NULL (-4)
#define CK_ERR_UNSUPPORTED (-5)
#define CK_ERR_DEVICE_TIMEOUT (-6)

/* ---- library ---- */
const char* ck_last_error(void);
int ck_abi_version(void);
int ck_check_device(void); /* 0 when the current device is sm_100 */
/* Library options (process-wide).  The one option that belongs to the interface:
 * "nvfp4_exact_div" = 1 makes the NVFP4 quantizer use plain IEEE divisions instead of the
 * shared-reciprocal sequence; the bytes are the same either way (the tests check that on the
 * device), only the speed differs.  The launchers' tuning knobs are listed in the library's
 * internal header csrc/ck_options.h; none of them changes a result's bytes beyond what that
 * header states.  Unknown names return CK_ERR_UNSUPPORTED. */
int ck_set_option(const char* name, int value);

/* ---- per-tensor FP8 ----
 * Replaces launch_quantize_fp8_kernel / launch_dequantize_fp8_kernel
 * (backends/cuda/dlpack_bindings.cpp:45-52, ops/per_tensor_quantize.cu:170-237).
 * scale: one device float.  Arithmetic: backends/eager/quantization.py:43-63. */
int launch_quantize_fp8_kernel(const void* input, void* output, const void* scale, int64_t numel,
                               int input_dtype_code, int output_dtype_code, ck_stream_t stream);

/* stochastic_rounding_fp8 (comfy_kitchen/backends/eager/quantization.py:66-114; reference kernel
 * backends/cuda/ops/per_tensor_quantize.cu:121-161, which overwrites the random bytes in place): input rounded
 * to fp16, then to FP8 with one random byte per element deciding the direction.  Byte-identical to the eager
 * function.  rng: numel bytes; output: numel bytes (E4M3 or E5M2 codes). */
int launch_stochastic_rounding_fp8_kernel(const void* input, const void* rng, void* output, int64_t numel,
                                          int input_dtype_code, int output_dtype_code, ck_stream_t stream);
int launch_dequantize_fp8_kernel(const void* input, void* output, const void* scale, int64_t numel,
                                 int input_dtype_code, int output_dtype_code, ck_stream_t stream);

/* ---- NVFP4 ----
 * Replaces launch_quantize_nvfp4_kernel / launch_dequantize_nvfp4_kernel
 * (dlpack_bindings.cpp:102-124, ops/quantize_nvfp4.cu:323-435).
 * input [orig_rows, orig_cols]; output bytes [num_rows, num_cols/2]; block_scales
 * tiled [roundup(num_rows,128), roundup(num_cols/16,4)]; num_* >= orig_* (the
 * excess reads as zero; pad_16x of the Python API).  epsilon is accepted and
 * ignored, as in the reference.  Arithmetic: backends/eager/quantization.py:117-221. */
int launch_quantize_nvfp4_kernel(const void* input, const void* global_scale, void* output, void* block_scales,
                                 int64_t num_rows, int64_t num_cols, int64_t orig_rows, int64_t orig_cols,
                                 float epsilon, int input_dtype_code, bool hi_first, ck_stream_t stream);
int launch_dequantize_nvfp4_kernel(const void* input, const void* global_scale, const void* block_scales,
                                   void* output, int64_t num_rows, int64_t num_cols, int output_dtype_code,
                                   bool hi_first, ck_stream_t stream);

/* NVFP4 quantize of the column concatenation [seg0 | seg1] (seg1 optional: cols1 = 0).  Element (row, c) of a
 * segment is read at  base + (c / group) * group_stride + row * row_stride + c % group  (elements of the input
 * dtype, bf16 or fp16), so a column slice of a wider matrix or attention's [heads, tokens, head_dim] output can be
 * quantized in place; act = 1 applies GELU (tanh form), rounded to the input dtype, first.  No counterpart in
 * the reference: it stands for gather / concatenate / activation kernels followed by
 * launch_quantize_nvfp4_kernel (whose bytes it reproduces when act = 0).  Widths, groups and strides are
 * multiples of 16 elements, bases 32-byte aligned; output and block_scales as for launch_quantize_nvfp4_kernel
 * with num_cols = cols0 + cols1 and no row padding. */
int launch_quantize_nvfp4_gather_kernel(const void* base0, int64_t cols0, int64_t group0, int64_t group_stride0,
                                        int64_t row_stride0, int act0, const void* base1, int64_t cols1,
                                        int64_t group1, int64_t group_stride1, int64_t row_stride1, int act1,
                                        const void* global_scale, void* output, void* block_scales,
                                        int64_t num_rows, int input_dtype_code, bool hi_first, ck_stream_t stream);

/* ---- MXFP8 ----
 * launch_quantize_mxfp8_kernel replaces the reference's entry point of that name
 * (dlpack_bindings.cpp:125-134, ops/quantize_mxfp8.cu:148-208).
 * launch_dequantize_mxfp8_kernel has no CUDA counterpart in the reference (eager
 * only: backends/eager/quantization.py:329-366). */
int launch_quantize_mxfp8_kernel(const void* input, void* output, void* block_scales, int64_t num_rows,
                                 int64_t num_cols, int64_t orig_rows, int64_t orig_cols, int input_dtype_code,
                                 ck_stream_t stream);
int launch_dequantize_mxfp8_kernel(const void* input, const void* block_scales, void* output, int64_t num_rows,
                                   int64_t num_cols, int output_dtype_code, ck_stream_t stream);

/* ---- block-scaled GEMMs:  D[M,N] = alpha * A[M,K] . W[N,K]^T + bias[N] ----
 * launch_cublas_gemm_blockwise_fp4_kernel keeps the reference's argument order
 * (weights first) and meaning (dlpack_bindings.cpp:60-74,
 * ops/cublas_gemm_nvfp4.cu:295-340): bias has the output dtype, workspace is
 * unused, accumulate must be false.  launch_scaled_mm_nvfp4_kernel is the same
 * kernel with activations first and an explicit bias dtype (fp32 allowed).
 * launch_scaled_mm_mxfp8_kernel has no CUDA counterpart in the reference (eager
 * forwards to torch: backends/eager/quantization.py:369-404).
 * K counts elements (multiple of 32); N multiple of 8; alpha is a device float
 * (NULL = 1). */
int launch_cublas_gemm_blockwise_fp4_kernel(const void* B_ptr, const void* B_decode_scale_ptr, const void* A_ptr,
                                            const void* A_decode_scale_ptr, void* D_ptr, const void* bias_ptr,
                                            int64_t M, int64_t N, int64_t K, const float* alpha_device_ptr,
                                            int out_dtype_code, void* workspace_ptr, bool accumulate,
                                            ck_stream_t stream);
int launch_scaled_mm_nvfp4_kernel(const void* A, const void* A_scale, const void* B, const void* B_scale, void* D,
                                  const void* bias, int bias_dtype_code, int64_t M, int64_t N, int64_t K,
                                  const float* alpha_device_ptr, int out_dtype_code, ck_stream_t stream);
/* launch_scaled_mm_nvfp4_kernel followed by D = residual + gate[n] * D in the same kernel (the residual update
 * of a transformer block; no counterpart in the reference).  residual: [M, N] in the output dtype (bf16 / fp16),
 * may be D itself; gate: [N] in the output dtype.  Bytes equal GEMM -> elementwise addcmul on the stored tensors. */
int launch_scaled_mm_nvfp4_residual_kernel(const void* A, const void* A_scale, const void* B, const void* B_scale,
                                           void* D, const void* bias, int bias_dtype_code, const void* residual,
                                           const void* gate, int64_t M, int64_t N, int64_t K,
                                           const float* alpha_device_ptr, int out_dtype_code, ck_stream_t stream);
/* launch_scaled_mm_nvfp4_kernel with its output scattered by rows over the ranks of a tensor-parallel group: the
 * reduce-scatter that follows a row-parallel GEMM, fused into the epilogue (tile rows go straight to the rank that
 * will sum them, over NVLink, while the main loop carries on).  Output row r is row row_offset + r of the group's
 * matrix; rows [bounds[d], bounds[d+1]) go to dests[d], a [bounds[d+1] - bounds[d], N] buffer in rank d's memory mapped
 * into this process, counted from bounds[d].  dests / bounds: HOST arrays (world pointers; world + 1 ascending row
 * numbers, multiples of 128 except the last); row_offset and M multiples of 32; 16-bit outputs.  No counterpart in the
 * reference (no multi-GPU code). */
int launch_scaled_mm_nvfp4_scatter_kernel(const void* A, const void* A_scale, const void* B, const void* B_scale,
                                          void* const* dests, const int64_t* bounds, int world, int64_t row_offset,
                                          const void* bias, int bias_dtype_code, int64_t M, int64_t N, int64_t K,
                                          const float* alpha_device_ptr, int out_dtype_code, ck_stream_t stream);
int launch_scaled_mm_mxfp8_kernel(const void* A, const void* A_scale, const void* B, const void* B_scale, void* D,
                                  const void* bias, int bias_dtype_code, int64_t M, int64_t N, int64_t K,
                                  int out_dtype_code, ck_stream_t stream);
/* Synchronises the device, reads and clears the GEMM kernels' status word.  Returns 0, or
 * CK_ERR_DEVICE_TIMEOUT when a bounded device-side wait ran out since the last call
 * (ck_last_error() names the wait and the CTA), or a positive cudaError_t. */
int ck_gemm_device_status(void);

/* ---- RoPE ----
 * Replaces launch_apply_rope_kernel (dlpack_bindings.cpp:75-101,
 * ops/apply_rope.cu:358-404).  x is [batch, dim1, dim2, head_dim] with the given
 * element strides (used for input and output alike); freqs is
 * [freqs_batch, freqs_dim1, freqs_dim2, head_dim/2, 2, 2], each leading dim 1
 * (broadcast) or >= x's.  xk / xk_out may both be NULL.
 * Arithmetic: backends/eager/rope.py:9-32. */
int launch_apply_rope_kernel(const void* xq, const void* xk, const void* freqs, void* xq_out, void* xk_out,
                             int64_t batch, int64_t dim1, int64_t dim2, int64_t head_dim, int64_t freqs_batch,
                             int64_t freqs_dim1, int64_t freqs_dim2, int64_t stride_x_batch, int64_t stride_x_dim1,
                             int64_t stride_x_dim2, int64_t stride_x_dim, int64_t stride_freqs_batch,
                             int64_t stride_freqs_dim1, int64_t stride_freqs_dim2, int64_t stride_freqs_dim,
                             int64_t stride_freqs_rot, int64_t stride_freqs_pair, int input_dtype_code,
                             int freqs_dtype_code, bool split_half, ck_stream_t stream);

/* Per-head RMSNorm of q and k + RoPE of both + relayout of q, k, v for attention, one pass.
 * No single counterpart in the reference: it composes apply_rope (backends/eager/rope.py:9-32)
 * with torch's rms_norm and the caller's permutes.  qkv: [tokens, >= 3*heads*128] with row_stride
 * elements between tokens, columns [q heads | k heads | v heads]; q_weight, k_weight: [128] in
 * qkv's dtype (bf16 or fp16); freqs: fp32 [total_tokens, 64, 2, 2]; q_out, k_out, v_out:
 * [heads, total_tokens, 128]; rows token_offset .. token_offset+tokens-1 of every head are written. */
int launch_qk_norm_rope_kernel(const void* qkv, int64_t row_stride, const void* q_weight, const void* k_weight,
                               const float* freqs, void* q_out, void* k_out, void* v_out, int64_t tokens,
                               int64_t heads, int64_t token_offset, int64_t total_tokens, float eps,
                               int dtype_code, ck_stream_t stream);

/* ---- AdaLN / RMSNorm ----
 * launch_adaln_kernel replaces the reference's entry point of that name
 * (dlpack_bindings.cpp:196-207, ops/adaln.cu:247-300): x, out [N, D]; scale
 * [N/scale_group, D]; shift [N/shift_group, D]; row r reads modulation row
 * r/group (backends/_modulation.py:12-57).
 * launch_rmsnorm_kernel and the two fused norm->quantize entry points have no
 * counterpart in the reference; their packed outputs equal launch_adaln_kernel
 * (or launch_rmsnorm_kernel) followed by the matching quantizer, byte for byte.
 * norm_kind: 0 = LayerNorm + (1+scale), shift; 1 = RMSNorm with weight `scale`
 * (one row, NULL = no weight) and no shift. */
int launch_adaln_kernel(const void* x, const void* scale, const void* shift, void* out, int64_t N, int64_t D,
                        int64_t scale_group, int64_t shift_group, float eps, int dtype_code, ck_stream_t stream);
int launch_rmsnorm_kernel(const void* x, const void* weight, void* out, int64_t N, int64_t D, float eps,
                          int dtype_code, ck_stream_t stream);
int launch_adaln_quantize_nvfp4_kernel(const void* x, const void* scale, const void* shift, const void* global_scale,
                                       void* output, void* block_scales, int64_t N, int64_t D, int64_t scale_group,
                                       int64_t shift_group, float eps, int dtype_code, bool hi_first, int norm_kind,
                                       ck_stream_t stream);
/* launch_adaln_quantize_nvfp4_kernel restricted to rows [row_begin, row_end) of the N rows, written at the places
 * the whole-tensor call writes them (a range ending at N also writes the scale buffer's padding rows).  The bytes
 * equal the whole-tensor call's whenever the launcher gives both the same number of warps per row, which it chooses
 * from the number of rows processed (two below 2368 rows, else one); otherwise the row statistics are summed in
 * another order and an activation may move by one rounding step.  For sequence-parallel callers; no counterpart in
 * the reference. */
int launch_adaln_quantize_nvfp4_rows_kernel(const void* x, const void* scale, const void* shift,
                                            const void* global_scale, void* output, void* block_scales, int64_t N,
                                            int64_t D, int64_t scale_group, int64_t shift_group, float eps,
                                            int dtype_code, bool hi_first, int norm_kind, int64_t row_begin,
                                            int64_t row_end, ck_stream_t stream);
int launch_adaln_quantize_mxfp8_kernel(const void* x, const void* scale, const void* shift, void* output,
                                       void* block_scales, int64_t N, int64_t D, int64_t scale_group,
                                       int64_t shift_group, float eps, int dtype_code, int norm_kind,
                                       ck_stream_t stream);
/* Synchronises the device, reads and clears the norm kernels' status word.  Returns 0, or
 * CK_ERR_DEVICE_TIMEOUT when a bounded device-side wait on a row copy ran out since the last
 * call (the rows concerned were not written), or a positive cudaError_t. */
int ck_norm_device_status(void);

/* ---- tensor-parallel exchange (no counterpart in the reference, which has no multi-GPU code) ----
 * Stands where a tensor-parallel port would call ncclAllReduce on the row-parallel GEMM's output and
 * then an elementwise kernel:  x <- x + gate * (sum over ranks of partial), on every rank, in one
 * kernel over NVLink peer memory.  Every rank launches it with the same arguments but its own `rank`.
 * partials / residuals / pads: HOST arrays of `world` device pointers, entry i being rank i's buffer
 * as mapped into this process (memory mapped for this device: CUDA virtual-memory handles, i.e. symmetric memory); partial and
 * residual are [rows, cols] of the 16-bit dtype; a pad is ck_tp_pad_bytes() bytes, zeroed once before
 * first use, written by the kernel only.  Rows below split_row use gate0, the others gate1 (each [cols];
 * gate1 NULL = gate0 for all).  mc_partial / mc_residual: the NVLink-switch multicast addresses of the same
 * two buffers (both or neither; NULL = plain peer loads and stores): with them the sum is formed inside the
 * switch (multimem.ld_reduce, fp32 accumulation, one rounding) and the result is broadcast by it (multimem.st).
 * blocks: grid size, the same on every rank (0 = default).  All ranks'
 * residual buffers end bit-identical.  Waits for peers are bounded (seconds); see ck_tp_device_status. */
int64_t ck_tp_pad_bytes(void);
int launch_tp_exchange_kernel(const void* const* partials, void* const* residuals, void* const* pads,
                              const void* mc_partial, void* mc_residual, int world, int rank, const void* gate0, const void* gate1, int64_t split_row, int64_t rows,
                              int64_t cols, int dtype_code, int blocks, ck_stream_t stream);
/* Sequence-parallel form (no counterpart in the reference): launch_tp_reduce_rows_kernel sums rows [row_lo, row_hi)
 * of all ranks' partial results and updates those rows of this rank's own residual buffer only (the ranks' row ranges
 * partition the matrix); launch_tp_gather_kernel then copies up to two byte ranges [lo, hi) (multiples of 16) of this
 * rank's buffer to the same offsets of every peer's buffer and waits until all peers have done the same -- e.g. the
 * quantized activation a rank computed for its rows.  bufs / pads: host arrays of `world` device pointers as above;
 * both kernels use the flag pad (different parts of it) and every rank must issue the same sequence of calls. */
int launch_tp_reduce_rows_kernel(const void* const* partials, void* const* residuals, void* const* pads, int world,
                                 int rank, const void* gate0, const void* gate1, int64_t split_row, int64_t rows,
                                 int64_t cols, int64_t row_lo, int64_t row_hi, int dtype_code, int blocks,
                                 ck_stream_t stream);
int launch_tp_gather_kernel(void* const* bufs, void* const* pads, int world, int rank, int64_t lo0, int64_t hi0,
                            int64_t lo1, int64_t hi1, int blocks, ck_stream_t stream);
/* No counterpart in the reference.  The one-rank exchange (residual <- residual + gate * partial) for callers
 * that must not allocate device memory at call time -- a runtime with a fixed arena, a plugin inside a pipeline
 * where cudaMalloc would synchronise: the flag pad the kernel needs lives in a device array inside the library
 * (34 816 bytes per GPU, held until exit) instead of being passed in.  blocks > 512 is refused with
 * CK_ERR_SHAPE.  The first call on a device resolves the array's address; make it outside stream capture.  All
 * calls on a device share the pad: keep them on one stream (calls that overlap on the GPU race on it). */
int launch_tp_exchange_noalloc_kernel(const void* partial, void* residual, const void* gate0, const void* gate1,
                                      int64_t split_row, int64_t rows, int64_t cols, int dtype_code, int blocks,
                                      ck_stream_t stream);
/* Synchronises the device, reads and clears the exchange kernel's status word: 0, or
 * CK_ERR_DEVICE_TIMEOUT when a wait for a peer ran out since the last call. */
int ck_tp_device_status(void);

#ifdef __cplusplus
}
#endif
#endif /* COMFY_KITCHEN_B200_H_ */
