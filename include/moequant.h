/*
 * moequant.h - C ABI of libmoequant_sm100.so, the sm_100a GPTQ engine.
 *
 * The reference project (IST-DASLab/MoE-Quant) is pure Python: it has no FFI.
 * Each entry point below replaces a Python function (or the Triton / cuBLAS /
 * cuSOLVER calls underneath it) and cites that function by file:line relative
 * to the MoE-Quant project root.  The reference-side binding is a ctypes stub
 * that passes tensor.data_ptr() values and the current CUDA stream.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller unless said otherwise;
 *     the library allocates no device memory (mq_*_workspace_bytes tells the
 *     caller how much scratch to pass);
 *   - matrices are row-major; "ld" arguments are in elements;
 *   - `stream` is a cudaStream_t passed as void*; all work is stream-ordered and
 *     no entry point synchronises the device;
 *   - the return value is an mq_status; mq_last_error() gives the text of the
 *     last non-zero status on the calling thread;
 *   - numerical failures (NaN Hessian, non-positive pivot) are never errors:
 *     they are written to a device-side mq_layer_flags word that the caller
 *     reads when convenient.
 */
#ifndef MOEQUANT_H_
#define MOEQUANT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MQ_ABI_VERSION 2

typedef enum {
  MQ_OK = 0,
  MQ_ERR_ARGUMENT = 1,    /* null pointer, negative size, bad enum            */
  MQ_ERR_ALIGNMENT = 2,   /* pointer or leading dimension not aligned enough  */
  MQ_ERR_UNSUPPORTED = 3, /* shape outside what the kernels handle            */
  MQ_ERR_WORKSPACE = 4,   /* workspace too small                              */
  MQ_ERR_CUDA = 5         /* a CUDA runtime/driver call failed                */
} mq_status;

typedef enum { MQ_F32 = 0, MQ_BF16 = 1, MQ_F16 = 2 } mq_dtype;

/* Arithmetic used for the dense contractions.
 *   MQ_MATH_FP32  : fp32 FMA on the CUDA cores (bit-for-bit the reference's
 *                   "TF32 off" arithmetic up to summation order).
 *   MQ_MATH_TENSOR: tcgen05 tensor cores with fp32 TMEM accumulators.  bf16/fp16
 *                   operands enter exactly; fp32 operands are split into up to
 *                   three bf16 planes whose cross products are accumulated
 *                   (`split` planes: 1 -> 1 product, 2 -> 3, 3 -> 6).          */
typedef enum { MQ_MATH_FP32 = 0, MQ_MATH_TENSOR = 1 } mq_math;

/* Flag that may be OR-ed into the `math` argument of mq_gptq_sweep and mq_quantize_layer (and of
 * their *_workspace_bytes): the caller processes several layers at once on different streams
 * (gptq.quantize_many).  The library then prefers launch shapes that occupy few SMs over the
 * lowest latency of a single layer: the sweep's tiles run one weight row per thread on R/64
 * SMs instead of sixteen lanes per row on R/8 CTAs, a CTA of a rank-128 strip update walks a whole
 * row of output tiles, a CTA of a panel solve takes 64 rows instead of 32.  Results are bit-identical with and without it. */
#define MQ_MATH_COMPACT 0x100

/* Device-side status of one layer, written by mq_hessian_prepare / mq_hinv_upper.
 * Mirrors GPTQ.issue_nan_hessian / issue_non_invertible (src/gptq.py:61-63). */
typedef struct {
  int32_t nan_hessian;     /* 1: H held a NaN and was replaced by I (src/gptq.py:141-143) */
  int32_t dead_channels;   /* number of diag(H)==0 channels fixed (src/gptq.py:145-146)   */
  int32_t zero_columns;    /* number of all-zero weight columns masked (src/gptq.py:224-231) */
  int32_t not_positive;    /* 0, or 1+index of the first non-positive pivot; the factor is
                              then replaced by I (src/gptq.py:236-240)                    */
} mq_layer_flags;

int mq_abi_version(void);
const char* mq_last_error(void);

/* Every device-side wait in the tensor-core kernels is bounded.  If one ever expires the
 * kernel records a non-zero code, frees its resources and returns; results of that call are
 * then invalid.  This copies the current device's code to *host_out (0 = healthy).  It
 * synchronises the device, so call it where a synchronisation is acceptable.  */
int mq_engine_fault(int* host_out);
/* Resets the current device's code to 0 after the caller has dealt with a fault (dropped the
 * results computed since, checked the device).  Synchronises the device.  */
int mq_engine_fault_clear(void);

/* ------------------------------------------------------------------ a2
 * H <- beta*H + alpha*X^T X, H (C,C) fp32 symmetric, X (m,C) of x_dtype.
 * Replaces GPTQ.update's  H.addmm_(X.T, X, beta, alpha)  (src/gptq.py:97-105).
 * The full matrix (both triangles) is written.  */
int mq_hessian_accum(const void* X, int x_dtype, int64_t m, int64_t C, int64_t ldx,
                     float* H, int64_t ldh, float beta, float alpha,
                     int math, int split, void* workspace, size_t workspace_bytes, void* stream);
size_t mq_hessian_accum_workspace_bytes(int x_dtype, int64_t m, int64_t C, int math, int split);

/* ------------------------------------------------------------------ the contraction engine by itself
 * C[m,n] = alpha * sum_k A[m,k] B[k,n] + beta * C[m,n] on fp32 operands with arbitrary element
 * strides (A[m,k] at A[m*a_rs + k*a_cs], B[k,n] at B[k*b_rs + n*b_cs]), C row-major.
 * This is the GEMM that stands in for every torch addmm_ on the path (src/gptq.py:103,
 * src/gptq_loop.py:148) and for the library factorisations' inner products; it is exported so
 * that it can be tested and timed alone.  upper_tiles_only skips 128x128 output tiles that lie
 * entirely below the diagonal.  */
int mq_gemm(const float* A, int64_t a_rs, int64_t a_cs, const float* B, int64_t b_rs, int64_t b_cs,
            float* C, int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha, float beta,
            int upper_tiles_only, int math, int split,
            void* workspace, size_t workspace_bytes, void* stream);
size_t mq_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int math, int split);

/* ------------------------------------------------------------------ a3 + a5 (first half)
 * In place on H (C,C) and on the fp32 working copy W (R,C):
 *   NaN anywhere in H -> H = I;  diag(H)==0 -> 1 and that W column -> 0
 *   (GPTQ.quantization_pre_step, src/gptq.py:140-152);
 *   all-zero W columns -> their H row/column = 0, diagonal = 1;
 *   H += rel_damp * mean(diag H) * I   (GPTQ._get_hessian_inverse, src/gptq.py:224-234).
 * W may be NULL (then R is ignored and no column is masked).
 * workspace: mq_hessian_prepare_workspace_bytes(C).  */
int mq_hessian_prepare(float* H, int64_t C, int64_t ldh, float* W, int64_t R, int64_t ldw,
                       float rel_damp, mq_layer_flags* flags,
                       void* workspace, size_t workspace_bytes, void* stream);
size_t mq_hessian_prepare_workspace_bytes(int64_t C);

/* ------------------------------------------------------------------ no counterpart in the reference
 * mq_hessian_prepare for callers that cannot supply scratch memory: a C host that only holds
 * the H and W pointers, a plug-in that must not call the allocator of the process it runs in,
 * or a path on which cudaMalloc (which synchronises the device) is off limits.  Same arguments
 * and results as mq_hessian_prepare minus the workspace; the channel lists live in a
 * static device array inside the library instead.
 *   - limit: C <= 32768 input channels (the array is about 256 KB per GPU, held until the
 *     process exits); larger C returns MQ_ERR_UNSUPPORTED and changes nothing;
 *   - the library makes no allocation and frees nothing in this call;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call outside any stream capture;
 *   - all calls on a device share the one array, which keeps what the previous call left
 *     (each call clears what it needs): two calls that overlap on the GPU, e.g. on two
 *     streams, race.  Serialise them.  */
int mq_hessian_prepare_noalloc(float* H, int64_t C, int64_t ldh, float* W, int64_t R, int64_t ldw,
                               float rel_damp, mq_layer_flags* flags, void* stream);

/* ------------------------------------------------------------------ a5 (second half)
 * Uhat <- rownormalise(chol_upper(H^-1)):  upper triangular, unit diagonal, zeros below.
 * Replaces inv_sym + torch.linalg.cholesky(upper=True) + div_ by the diagonal
 * (src/linalg_utils.py:8-12, src/gptq.py:236-242) with one reverse Cholesky
 * H = T T^T (T upper) followed by the inverse of the unit-diagonal factor.
 * H is destroyed (its upper triangle ends up holding the scaled factor).
 * diag_out (optional, C floats) receives diag(T); H^-1 = Uhat^T diag(T)^-2 Uhat.
 * A non-positive pivot sets flags->not_positive and yields Uhat = I.  */
int mq_hinv_upper(float* H, int64_t C, int64_t ldh, float* Uhat, int64_t ldu, float* diag_out,
                  int math, int split, mq_layer_flags* flags,
                  void* workspace, size_t workspace_bytes, void* stream);
size_t mq_hinv_upper_workspace_bytes(int64_t C, int math, int split);

/* The first half of mq_hinv_upper alone: H (damped) -> Utilde = T diag(T)^-1 in place (unit upper
 * triangular, zeros below), with H = T T^T; diag_out (optional, C floats) receives diag(T).
 * Utilde is the inverse of Uhat.  mq_gptq_sweep accepts it directly (W_original != NULL), which
 * saves the triangular inverse: that is what mq_quantize_layer does.  Non-positive pivot:
 * flags->not_positive is set and the result is I.
 * workspace: mq_chol_unit_factor_workspace_bytes(C, math, split).  */
int mq_chol_unit_factor(float* H, int64_t C, int64_t ldh, float* diag_out, int math, int split,
                        mq_layer_flags* flags, void* workspace, size_t workspace_bytes, void* stream);
size_t mq_chol_unit_factor_workspace_bytes(int64_t C, int math, int split);

/* ------------------------------------------------------------------ a4
 * scale[r, j] = round_to(out_dtype, (2/maxq) * max|W[r, j*g:(j+1)*g]| + 1e-12), kept as fp32.
 * Symmetric grid of find_quantization_meta / get_quantization_grid
 * (src/quant_utils.py:75-101, 195-240); zero is the constant (maxq+1)/2.  */
int mq_absmax_scales(const float* W, int64_t R, int64_t C, int64_t ldw, int64_t group,
                     int bits, int out_dtype, float* scale, void* stream);

/* MSE refinement of the symmetric grid (QuantizationScale.MSE, src/quant_utils.py:104-192, 218-230):
 * every scale[r, j] (as written by mq_absmax_scales, rounded through out_dtype) is replaced by
 * round_to(out_dtype, scale * shrink[i*]) where i* minimises
 *   sum_c | dequant(quant(W[r, c]; round_to(out_dtype, scale * shrink[i]))) - W[r, c] |^norm
 * over the group.  shrink: n_shrink fp32 factors on the device (the reference uses
 * linspace(1, 0.2, 100)); norm 2.4 in the reference.  */
int mq_mse_scales(const float* W, int64_t R, int64_t C, int64_t ldw, int64_t group, int bits,
                  int out_dtype, const float* shrink, int n_shrink, float norm, float* scale,
                  void* stream);

/* ------------------------------------------------------------------ a6 + a7 + a8
 * GPTQ column sweep over W (R,C) fp32 (destroyed), given Uhat (C,C) upper/unit.
 * Replaces gptq_loop / quantize_error_triton_kernel / addvv_triton_kernel / the lazy
 * addmm_ (src/gptq_loop.py:12-225) and the transposes at src/gptq.py:191-199.
 *   scale, zero : element (r, c) is  base[r*row_stride + (c/group)*group_stride];
 *                 zero may be NULL (then (maxq+1)/2 is used).
 *   codes       : (R,C) uint8 out, row-major, values 0..maxq.
 *   packed      : optional (R, C/8) int32 out: the same codes in the compressed-tensors layout of
 *                 mq_pack_int4 (pack_quantized_model.py:57-75), written by the sweep itself so
 *                 that no packing pass reads the codes back.  Needs bits == 4 and zero == NULL.
 *   dequantized : optional (R,C) out of out_dtype holding round_to(out_dtype,(q-zero)*scale).
 *   out_dtype   : the layer dtype that dequantized values are rounded through inside the
 *                 sweep (src/quant_utils.py:37-49).
 *   W_original  : NULL for the reference's recurrence (Uhat given).  Otherwise a second, untouched
 *                 fp32 copy of the weights (ldwo) and `Uhat` must hold the unit factor Utilde of
 *                 mq_chol_unit_factor: the sweep then propagates -(y - w_original) against Utilde,
 *                 which yields the same running weights without ever inverting the factor.
 * workspace: mq_gptq_sweep_workspace_bytes(R, C, math, split).  */
int mq_gptq_sweep(float* W, int64_t R, int64_t C, int64_t ldw,
                  const float* Uhat, int64_t ldu,
                  const float* scale, const float* zero, int64_t group,
                  int64_t row_stride, int64_t group_stride,
                  int bits, int out_dtype,
                  uint8_t* codes, int32_t* packed, void* dequantized, const float* W_original, int64_t ldwo,
                  int math, int split, void* workspace, size_t workspace_bytes, void* stream);
size_t mq_gptq_sweep_workspace_bytes(int64_t R, int64_t C, int math, int split);

/* ------------------------------------------------------------------ a3..a8 in one call
 * GPTQ.quantize(bits) for one symmetric layer whose Hessian is complete
 * (src/gptq.py:122-218 without the collectives): clone W to fp32, prepare H (in place,
 * it ends up damped like the reference's handle.H), scales, Uhat, sweep.
 *   Wsrc (R,C) of w_dtype is not modified.
 *   scale_out (R, C/group) fp32 values already rounded through w_dtype.
 *   packed (optional, NULL or n_tied pointers): (R, C/8) int32 words per layer, see mq_gptq_sweep.
 *   n_tied > 1: Wsrc/codes/packed/scale_out/dequantized are arrays of n_tied device pointers
 *   passed from HOST memory; the layers share H (tied gate_proj/up_proj handles,
 *   quant.py:258-262) and therefore one factorisation.  With n_tied == 1 the same
 *   arguments are still pointer arrays of length 1.
 * workspace: mq_quantize_layer_workspace_bytes(...).  */
int mq_quantize_layer(const void* const* Wsrc, int w_dtype, int n_tied, int64_t R, int64_t C,
                      float* H, int64_t ldh, int64_t group, int bits, float rel_damp,
                      uint8_t* const* codes, int32_t* const* packed, float* const* scale_out,
                      void* const* dequantized,
                      mq_layer_flags* flags, int math, int split_hinv, int split_sweep,
                      void* workspace, size_t workspace_bytes, void* stream);
size_t mq_quantize_layer_workspace_bytes(int n_tied, int64_t R, int64_t C, int math,
                                         int split_hinv, int split_sweep);

/* ------------------------------------------------------------------ a10
 * out[r,c] = (codes[r,c] - zero[r, c/group]) * scale[r, c/group], rounded to out_dtype.
 * dequantize_linear_weight (src/quant_utils.py:243-256).  scale and zero are (R, C/group)
 * fp32; zero may be NULL, meaning the symmetric constant (maxq+1)/2.  */
int mq_dequantize(const uint8_t* codes, int64_t R, int64_t C, const float* scale, const float* zero,
                  int64_t group, int bits, int out_dtype, void* out, void* stream);

/* sum over (r,c) of (A H)[r,c] * A[r,c] for A (R,C) fp32 and H (C,C) fp32, written to *out
 * (one double on the device).  Numerator (A = q - w) and denominator (A = w) of
 * get_relative_mse_error (src/quant_utils.py:259-264), the metric quant.py:314-316 logs
 * after every layer.  workspace: mq_quadratic_form_workspace_bytes(R, C, math, split).  */
int mq_quadratic_form(const float* A, int64_t R, int64_t C, int64_t lda, const float* H, int64_t ldh,
                      double* out, int math, int split, void* workspace, size_t workspace_bytes,
                      void* stream);
size_t mq_quadratic_form_workspace_bytes(int64_t R, int64_t C, int math, int split);

/* ------------------------------------------------------------------ a11
 * compressed-tensors int4 -> int32 packing of pack_weight / pack_to_int32
 * (pack_quantized_model.py:57-75): nibble = codes - zero + 8, word k of a row holds
 * columns 8k..8k+7, column 8k+i at bits 4i..4i+3, tail columns padded with nibble 0.
 *   zero_i8 : optional (R, C/group) int8 zero points; NULL means 8 (symmetric).
 *   packed  : (R, ceil(C/8)) int32 out.  */
int mq_pack_int4(const uint8_t* codes, int64_t R, int64_t C, const int8_t* zero_i8, int64_t group,
                 int32_t* packed, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOEQUANT_H_ */
