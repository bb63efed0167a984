/*
 * aiter_b200 - C ABI of the B200 (sm_100a) quantised-GEMM library.
 *
 * Every entry point mirrors, name for name and argument for argument, the C-ABI / pybind
 * function the reference binds for the same job; the reference location is cited beside each
 * declaration (paths inside the reference project).  Conventions (reference:
 * csrc/include/aiter_ctypes_error.h:60-150, aiter/jit/core.py:1457-1553):
 *   - tensors travel as `aiter_tensor_t*` (160-byte POD, strides in elements, NULL = absent);
 *   - python int -> int64-compatible `int`, bool -> int, str -> const char* (NULL = absent);
 *   - the CUDA stream is the trailing `void*` argument (a cudaStream_t);
 *   - the return value is 0 on success and -1 on error; the message is kept per thread and read
 *     with aiter_get_last_error(); no C++ exception crosses the boundary;
 *   - the caller owns every buffer, outputs included; launches are asynchronous on the stream.
 */
#ifndef AITER_B200_H
#define AITER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* reference: csrc/include/aiter_enum.h:34-50 (same numbering) */
typedef enum
{
    AITER_DTYPE_fp8      = 0,
    AITER_DTYPE_fp8_e8m0 = 1,
    AITER_DTYPE_fp16     = 2,
    AITER_DTYPE_bf16     = 3,
    AITER_DTYPE_fp32     = 4,
    AITER_DTYPE_i4x2     = 5,
    AITER_DTYPE_fp4x2    = 6,
    AITER_DTYPE_u32      = 7,
    AITER_DTYPE_i32      = 8,
    AITER_DTYPE_i16      = 9,
    AITER_DTYPE_i8       = 10,
    AITER_DTYPE_u8       = 11,
    AITER_DTYPE_i64      = 12,
    AITER_DTYPE_u64      = 13
} AiterDtype;

/* reference: csrc/include/aiter_tensor.h:8-17; python mirror aiter/utility/aiter_types.py:68-88 */
typedef struct aiter_tensor_t
{
    void* ptr;
    size_t numel_;
    int ndim;
    int64_t shape[8];
    int64_t strides[8];
    AiterDtype dtype_;
    int device_id; /* -1 = host memory */
} aiter_tensor_t;

#define AITER_B200_API __attribute__((visibility("default")))

/* ---- error bridge: csrc/include/aiter_ctypes_error.h:60-77 ---- */
AITER_B200_API int aiter_ctypes_abi_version(void); /* returns 2 */
AITER_B200_API const char* aiter_get_last_error(void);
AITER_B200_API void aiter_clear_last_error(void);

/* ---- M bucket for tuned-table look-ups: csrc/py_itfs_cu/gemm_common.cu:12-41 ---- */
AITER_B200_API int getPaddedM(int M, int N, int K, int gl);

/* ---- MXFP4 x MXFP4 -> bf16.  csrc/py_itfs_cu/asm_gemm_a4w4.cu:158-173
 * A [M,K/2] packed e2m1, B [N,K/2] packed e2m1 ((16,16)-shuffled when bpreshuffle != 0),
 * A_scale / B_scale e8m0 in the e8m0_shuffle layout, out [>=M, N] bf16, bias fp32 [1,N] or NULL,
 * out = alpha * A.B^T + beta * bias, split-K = 2^log2_k_split (0 = none, <0 = library's choice). */
AITER_B200_API int gemm_a4w4_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* A_scale,
                                 aiter_tensor_t* B_scale, aiter_tensor_t* out, const char* kernelName,
                                 aiter_tensor_t* bias, float alpha, float beta, int bpreshuffle,
                                 int log2_k_split, void* stream);

/* ---- same math through the reference's second back-end names.
 * csrc/include/rocm_ops.hpp:713-723, csrc/ck_gemm_a4w4_blockscale/gemm_a4w4_blockscale.cu:69-93 */
AITER_B200_API int gemm_a4w4_blockscale(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                        aiter_tensor_t* w_scale, aiter_tensor_t* Out, int splitK,
                                        const char* kernelName, void* stream);
AITER_B200_API int gemm_a4w4_blockscale_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                             aiter_tensor_t* w_scale, aiter_tensor_t* Out, int kernelId,
                                             int splitK, void* stream);

/* ---- MXFP8 x MXFP8 and MXFP8 x MXFP4 -> bf16.  csrc/py_itfs_cu/asm_mxfp8fp4gemm.cu:272-302
 * A [M,K] e4m3 ((m/2,k/128,2,128)-tiled when a_preshuffle != 0), B 16x16-byte tile transposed,
 * scales e8m0 in the (m/32,k/4,32,4) layout, out [M,N] bf16, K % 128 == 0. */
AITER_B200_API int mxfp8_mxfp8_gemm_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA,
                                        aiter_tensor_t* ScaleB, aiter_tensor_t* out, const char* kernelName,
                                        int a_preshuffle, void* stream);
AITER_B200_API int mxfp8_mxfp4_gemm_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA,
                                        aiter_tensor_t* ScaleB, aiter_tensor_t* out, const char* kernelName,
                                        int a_preshuffle, void* stream);

/* ---- FP8 x FP8 with fp32 scales per 128-wide K block -> bf16.  csrc/include/rocm_ops.hpp:725-765,
 * csrc/ck_gemm_a8w8_blockscale/gemm_a8w8_blockscale.cu:82-112, csrc/py_itfs_cu/asm_a8w8_blockscale_bpreshuffle.cu:59-73.
 * XQ [M,K] e4m3, WQ [N,K] e4m3 (plain, or (16,16)-shuffled for the _bpreshuffle forms), x_scale [M,K/128] fp32
 * (stored K-block-major for the _bpreshuffle forms), w_scale [ceil(N/128),K/128] fp32, Out [M,N] bf16, fp16 or fp32, K % 128 == 0.
 * One kernel instance serves the path: kernelName / splitK are accepted and ignored, kernelId must be 0. */
AITER_B200_API int gemm_a8w8_blockscale(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                        aiter_tensor_t* w_scale, aiter_tensor_t* Out, int splitK,
                                        const char* kernelName, void* stream);
AITER_B200_API int gemm_a8w8_blockscale_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                             aiter_tensor_t* w_scale, aiter_tensor_t* Out, int kernelId,
                                             int splitK, void* stream);
AITER_B200_API int gemm_a8w8_blockscale_bpreshuffle(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                                    aiter_tensor_t* w_scale, aiter_tensor_t* Out, int splitK,
                                                    const char* kernelName, void* stream);
AITER_B200_API int gemm_a8w8_blockscale_bpreshuffle_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ,
                                                         aiter_tensor_t* x_scale, aiter_tensor_t* w_scale,
                                                         aiter_tensor_t* Out, int kernelId, int splitK, void* stream);
/* The same arithmetic under the reference's other back-end names, each with its own argument order
 * (csrc/include/rocm_ops.hpp:749-821 for the CK-tile forms; aiter/ops/gemm_op_a8w8.py:342-381 for the assembly forms:
 * flatmm_a8w8_blockscale_asm takes a row-major weight, gemm_a8w8_blockscale_bpreshuffle_asm the (16,16)-shuffled one and
 * accepts no bias here). */
AITER_B200_API int gemm_a8w8_blockscale_cktile(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale, aiter_tensor_t* w_scale,
                                               aiter_tensor_t* Out, int preshuffleB, int splitK, const char* kernelName, void* stream);
AITER_B200_API int gemm_a8w8_blockscale_cktile_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                                    aiter_tensor_t* w_scale, aiter_tensor_t* Out, int kernelId, int splitK,
                                                    int preshuffleB, void* stream);
AITER_B200_API int gemm_a8w8_blockscale_bpreshuffle_cktile(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                                           aiter_tensor_t* w_scale, aiter_tensor_t* Out, int preshuffleB,
                                                           const char* kernelName, void* stream);
AITER_B200_API int gemm_a8w8_blockscale_bpreshuffle_cktile_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale,
                                                                aiter_tensor_t* w_scale, aiter_tensor_t* Out, int kernelId, int splitK,
                                                                int preshuffleB, void* stream);
AITER_B200_API int flatmm_a8w8_blockscale_asm(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* x_scale, aiter_tensor_t* w_scale,
                                              aiter_tensor_t* out, void* stream);
AITER_B200_API int gemm_a8w8_blockscale_bpreshuffle_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* out, aiter_tensor_t* A_scale,
                                                        aiter_tensor_t* B_scale, aiter_tensor_t* bias, int splitK, const char* kernelName,
                                                        int bpreshuffle, aiter_tensor_t* zero_bias_buf, void* stream);


/* ---- MXFP4 x MXFP4 with the (m/32,k/4,32,4) scale layout (the F4GEMM entry point).  csrc/py_itfs_cu/asm_f4gemm.cu:396-412,
 * Python side aiter/ops/gemm_op_a4w4.py:288-407,457-567 (gemm_mxfp4_asm, gemm_a4w4o4, gemm_a4w4o8).
 * A [M,K/2] and B [N,K/2] packed e2m1; B, and A when a_preshuffle != 0, as 16x16-byte tiles.  The output tensor selects the form:
 *   bf16 [M,N], out_scale NULL;
 *   fp4x2 / uint8 [M,N/2], out_scale NULL: packed e2m1 of the product WITHOUT the block scales (the reference's
 *     fp4-output kernel is its "noscale" variant), round to nearest even, saturating;
 *   fp8 [M,N] + out_scale [M,N/128] e8m0: e4m3 data with one RoundUp(amax/448) scale per 128 output columns, the scale
 *     bytes in the packed (M/64, N/128, 16, 4) order; needs M % 64 == 0.
 * The low-precision forms need N % 128 == 0. */
AITER_B200_API int mxfp4_gemm_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA,
                                  aiter_tensor_t* ScaleB, aiter_tensor_t* out, aiter_tensor_t* out_scale,
                                  const char* kernelName, int a_preshuffle, void* stream);

/* ---- NVFP4 x NVFP4: the same entry point with e4m3 scales per 16 elements and two per-tensor scales.
 * Python side aiter/ops/gemm_op_a4w4.py:305-321,410-443 (_nvfp4_gemm_asm, gemm_nvfp4_asm); reference
 * arithmetic op_tests/test_f4gemm.py:122-133: out = float(gA) * float(gB) * (deq A)(deq B)^T, deq x = e2m1(x) * e4m3(scale).
 * ScaleA [M, K/16], ScaleB [N, K/16]: non-negative e4m3 bytes (fp8 or uint8 tensors) in tiles of 32 rows x 8 scales
 * (aiter/ops/shuffle.py:293-316 with intype 8); rows padded to a multiple of 32; K % 256 == 0.
 * Output forms as for mxfp4_gemm_asm; the packed-fp4 form drops the block scales and keeps the per-tensor ones. */
AITER_B200_API int nvfp4_gemm_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA,
                                  aiter_tensor_t* ScaleB, float GlobalScaleA, float GlobalScaleB,
                                  aiter_tensor_t* out, aiter_tensor_t* out_scale, const char* kernelName,
                                  int a_preshuffle, void* stream);

/* ---- bf16 x bf16, fp32 accumulate.  aiter/ops/gemm_op_a16w16.py:12-26 (asm form),
 * csrc/opus_gemm/include/opus_gemm.h:16-39 and csrc/opus_gemm/opus_gemm.cu:133-209,294-350 (opus forms).
 * A [M,K], B [N,K] ((16,16)-shuffled when bpreshuffle != 0), out [M,N] bf16 or fp32 (fp32 is stored straight from the
 * accumulator), bias bf16/fp32 [N] or NULL.
 * The opus forms take [batch,M,K] x [batch,N,K] -> [batch,M,N] as ONE launch (the batch is a tile coordinate), bias [N] or
 * [batch,N]; splitK: log2 of the K split, <0 = auto.  opus_gemm with fp8 operands, x_scale [batch,M,K/128] and w_scale
 * [batch,N/128,K/128] (fp32) is the reference's a8w8_scale pipeline: fp32 output, no bias, served by the
 * fp32-blockscale kernels (one launch per batch entry). */
AITER_B200_API int gemm_a16w16_asm(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* out,
                                   aiter_tensor_t* semaphore, aiter_tensor_t* bias, int splitK,
                                   const char* kernelName, int bpreshuffle, void* stream);
AITER_B200_API int opus_gemm_a16w16_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* Y,
                                         aiter_tensor_t* bias, int kernelId, int splitK, void* stream);
AITER_B200_API int opus_gemm(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* Y,
                             aiter_tensor_t* group_layout, aiter_tensor_t* x_scale, aiter_tensor_t* w_scale,
                             aiter_tensor_t* bias, void* stream);
AITER_B200_API int opus_gemm_workspace_init(void);

/* ---- batched bf16: out[b,M,N] = XQ[b,M,K] WQ[b,N,K]^T, bf16 or fp16 out, the whole batch in one launch.
 * csrc/ck_batched_gemm_bf16/batched_gemm_bf16.cu:126-148 (pybind there: csrc/include/rocm_ops.hpp:249-262), Python side
 * aiter/ops/batched_gemm_op_bf16.py:27-148.  As in the reference the bias is only checked (same dtype as out), never
 * added, and splitK of the plain form is accepted and ignored; the _tune form takes a kernel id of the menu and log2 of
 * the K split.  K-contiguous operands; row and batch strides multiples of 8 elements (a transposed [M,b,K] view works). */
AITER_B200_API int batched_gemm_bf16(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* out, aiter_tensor_t* bias,
                                     int splitK, void* stream);
AITER_B200_API int batched_gemm_bf16_tune(aiter_tensor_t* XQ, aiter_tensor_t* WQ, aiter_tensor_t* out, int kernelId,
                                          int splitK, void* stream);

/* ---- MXFP8 x MXFP8 -> bf16 without any device allocation.  No counterpart in the reference.
 * For callers that must not call cudaMalloc (a pre-sized arena, a plugin that may not touch the host's
 * allocator, a latency-critical loop): same arguments and results as mxfp8_mxfp8_gemm_asm, but the split-K
 * partial sums, ticket counters and status record live in a fixed 8 MiB + 32 KiB array inside the library
 * image (held by every GPU that loads the library until the process exits).  A shape whose split-K partials
 * exceed 8 MiB, or that has more than 4096 output tiles under split-K, is refused with an error.  The first
 * call on a device looks up the array's address (no allocation) and should be made before any stream
 * capture.  All calls share the array: calls that overlap on the GPU race. log2_k_split < 0: library's choice. */
AITER_B200_API int aiter_b200_gemm_a8w8_mxfp8_noalloc(aiter_tensor_t* A, aiter_tensor_t* B, aiter_tensor_t* ScaleA,
                                                      aiter_tensor_t* ScaleB, aiter_tensor_t* out, int a_preshuffle,
                                                      int log2_k_split, void* stream);
/* The status record of the entry point above (it lives in the same fixed array, not in the record
 * aiter_b200_device_status reads): 4 words, all zero unless a bounded wait inside one of its kernels ran out
 * (code, block, split, iteration).  Synchronises the device, copies the record out and clears it; allocates
 * nothing.  A record stays in place across later calls until it is fetched here.  No counterpart in the reference. */
AITER_B200_API int aiter_b200_noalloc_status(int device, unsigned int out_words[4]);

/* ---- dynamic 1x32 MX quantisation of activations (the step in front of the GEMM) ----
 * Replaces dynamic_per_group_scaled_quant (csrc/include/quant.h:29-35, kernel csrc/kernels/quant_mxfp4.cu:88-212;
 * Python: per_1x32_mx_quant_hip, aiter/ops/quant.py:486-597).  input [M, K] bf16 / fp16; out [M, K/2] fp4x2 / uint8
 * (MXFP4) or [M, K] fp8 (MXFP8); scales: e8m0 bytes, RoundUp(amax / max) per 32 elements.
 * shuffle_scale 0: scales [M, K/32]; 1: e8m0_shuffle order in a [pad256(M), pad8(K/32)] array (what gemm_a4w4 takes);
 * 2 (no counterpart in the reference): the (m/32, k/4, 32, 4) order in a [pad32(M), K/32] array, what the MXFP8 /
 * mixed GEMM entry points take.  group_size must be 32; num_rows must be NULL and num_rows_factor 1. */
AITER_B200_API int dynamic_per_group_scaled_quant(aiter_tensor_t* out, aiter_tensor_t* input, aiter_tensor_t* scales,
                                                  int group_size, int shuffle_scale, aiter_tensor_t* num_rows,
                                                  int num_rows_factor, void* stream);

/* ---- library state ---- */
/* Copies the 4-word device status record of `device` (0 = healthy; non-zero = a bounded wait
 * inside a kernel expired: code, block, split, iteration) and clears it.  Synchronises the device.
 * While a non-zero record is pending every GEMM entry point on that device fails with a message that
 * names the code (the kernels mirror it into a pinned host word the launcher reads), so a caller that
 * never polls still learns of an incomplete output at its next call. */
AITER_B200_API int aiter_b200_device_status(int device, unsigned int out_words[4]);
/* Test and diagnosis hook (no counterpart in the reference): the wall-time bound of every in-kernel wait on
 * `device`, 1 ms .. 10 s (default 1 s), and a switch that makes the scale producer of the MX GEMM kernel issue
 * nothing, so that the waits behind it run out after that bound, the kernel records its status and returns by
 * itself.  Used to exercise the time-out path without faulting or hanging anything.  Synchronises the device. */
AITER_B200_API int aiter_b200_debug_wait_control(int device, unsigned long long limit_ns, int withhold_scales);
/* Human-readable list of the kernel configurations behind `kernelName`/`kernelId`. */
AITER_B200_API const char* aiter_b200_kernel_list(void);
/* Name of the configuration the heuristic picks for a problem (kind: 0 bf16, 1 mxfp8, 2 mxfp4, 3 mxfp8 x mxfp4). */
AITER_B200_API const char* aiter_b200_heuristic_name(int kind, int M, int N, int K, int* log2_splitk);
/* Number of kernel launches issued by this library since load (all threads). */
AITER_B200_API unsigned long long aiter_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* AITER_B200_H */
