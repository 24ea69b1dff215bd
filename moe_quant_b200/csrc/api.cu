// C-ABI entry points that tie the kernels together: Hessian accumulation and the
// whole-layer GPTQ.quantize() replacement.  Host-side orchestration only; every
// launch goes to the caller's stream and nothing here synchronises.
#include <stdarg.h>

#include "engine.cuh"

namespace mq {

static thread_local char g_error[512] = "";
long long g_launches = 0;

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

// defined in the other translation units
int launch_to_fp32(const void* src, int dtype, float* dst, int64_t n, cudaStream_t st);
size_t hinv_workspace_bytes(int64_t C, int math, int split);
size_t factor_workspace_bytes(int64_t C, int math, int split);
int hinv_upper(float* H, int64_t C, int64_t ldh, float* Uhat, int64_t ldu, float* diag_out, int math, int split, mq_layer_flags* flags,
               Workspace& ws, cudaStream_t st);
size_t sweep_workspace_bytes(int64_t R, int64_t C, int math, int split);
int gptq_sweep(float* W, int64_t R, int64_t C, int64_t ldw, const float* Uhat, int64_t ldu, const float* scale,
               const float* zero, int64_t group, int64_t s_rs, int64_t s_gs, int bits, int out_dtype, uint8_t* codes,
               void* deq, const float* Worig, int64_t ldwo, int math, int split, Workspace& ws, cudaStream_t st,
               const float* col_div, int32_t* packed);
int chol_unit_factor(float* H, int64_t C, int64_t ldh, float* diag, int math, int split, mq_layer_flags* flags,
                     Workspace& ws, cudaStream_t st, bool upper_only, bool unscaled);
int hessian_accum_tensor(const void* X, int x_dtype, int64_t m, int64_t C, int64_t ldx, float* H, int64_t ldh, float beta,
                         float alpha, int split, Workspace& ws, cudaStream_t st);
size_t hessian_accum_tensor_workspace_bytes(int x_dtype, int64_t m, int64_t C, int split);

}  // namespace mq

extern "C" int mq_abi_version(void) { return MQ_ABI_VERSION; }
extern "C" const char* mq_last_error(void) { return mq::g_error; }

// ---------------------------------------------------------------------------- a2
extern "C" size_t mq_hessian_accum_workspace_bytes(int x_dtype, int64_t m, int64_t C, int math, int split) {
  if (math == MQ_MATH_TENSOR) return mq::hessian_accum_tensor_workspace_bytes(x_dtype, m, C, split);
  return 0;
}

extern "C" int mq_hessian_accum(const void* X, int x_dtype, int64_t m, int64_t C, int64_t ldx, float* H, int64_t ldh,
                                float beta, float alpha, int math, int split, void* workspace, size_t workspace_bytes,
                                void* stream) {
  using namespace mq;
  MQ_REQUIRE(H, MQ_ERR_ARGUMENT, "mq_hessian_accum: null H");
  MQ_REQUIRE(m >= 0 && C > 0 && ldh >= C, MQ_ERR_ARGUMENT, "mq_hessian_accum: bad shape m=%lld C=%lld ldh=%lld", (long long)m,
             (long long)C, (long long)ldh);
  MQ_REQUIRE(m == 0 || (X && ldx >= C), MQ_ERR_ARGUMENT, "mq_hessian_accum: bad X or ldx=%lld", (long long)ldx);
  MQ_REQUIRE(valid_dtype(x_dtype), MQ_ERR_ARGUMENT, "mq_hessian_accum: bad dtype %d", x_dtype);
  MQ_REQUIRE(math == MQ_MATH_FP32 || math == MQ_MATH_TENSOR, MQ_ERR_ARGUMENT, "mq_hessian_accum: bad math %d", math);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Workspace ws(workspace, workspace_bytes);
  if (math == MQ_MATH_TENSOR) return hessian_accum_tensor(X, x_dtype, m, C, ldx, H, ldh, beta, alpha, split, ws, st);
  GemmDesc g;
  g.A = X; g.a_rs = 1; g.a_cs = ldx;   // A = X^T : A[c, t] = X[t, c]
  g.B = X; g.b_rs = ldx; g.b_cs = 1;   // B = X
  g.C = H; g.ldc = ldh;
  g.M = (int)C; g.N = (int)C; g.K = (int)m;
  g.alpha = alpha; g.beta = beta;
  g.upper_tiles_only = 1;
  MQ_TRY(gemm_simt(g, x_dtype, st));
  return mirror_upper_to_lower(H, C, ldh, st);
}

// ---------------------------------------------------------------------------- the GEMM engine by itself
extern "C" size_t mq_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int math, int split) {
  return mq::engine_workspace_bytes(M, N, K, math, split);
}

extern "C" int mq_gemm(const float* A, int64_t a_rs, int64_t a_cs, const float* B, int64_t b_rs, int64_t b_cs, float* C,
                       int64_t ldc, int64_t M, int64_t N, int64_t K, float alpha, float beta, int upper_tiles_only,
                       int math, int split, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace mq;
  MQ_REQUIRE(A && B && C, MQ_ERR_ARGUMENT, "mq_gemm: null pointer");
  MQ_REQUIRE(M > 0 && N > 0 && K >= 0 && ldc >= N, MQ_ERR_ARGUMENT, "mq_gemm: bad shape M=%lld N=%lld K=%lld ldc=%lld",
             (long long)M, (long long)N, (long long)K, (long long)ldc);
  MQ_REQUIRE(math == MQ_MATH_FP32 || math == MQ_MATH_TENSOR, MQ_ERR_ARGUMENT, "mq_gemm: bad math %d", math);
  GemmDesc g;
  g.A = A; g.a_rs = a_rs; g.a_cs = a_cs;
  g.B = B; g.b_rs = b_rs; g.b_cs = b_cs;
  g.C = C; g.ldc = ldc;
  g.M = (int)M; g.N = (int)N; g.K = (int)K;
  g.alpha = alpha; g.beta = beta;
  g.upper_tiles_only = upper_tiles_only;
  Workspace ws(workspace, workspace_bytes);
  Engine eng(math, split, ws, static_cast<cudaStream_t>(stream));
  return eng.gemm(g);
}

// ---------------------------------------------------------------------------- a3..a8
namespace mq {
static size_t layer_fixed_bytes(int n_tied, int64_t R, int64_t C) {
  size_t b = 0;
  b += align_up((size_t)C * C * sizeof(float), 256);                        // unit factor of the damped Hessian
  b += align_up((size_t)C * sizeof(float), 256);                            // its diagonal scaling
  b += 2 * (size_t)n_tied * align_up((size_t)R * C * sizeof(float), 256);   // fp32 weights: original and running
  b += mq_hessian_prepare_workspace_bytes(C);
  return b;
}
}  // namespace mq

namespace mq {
// dst[r, c] = src[r, c] for c from the start of row r's 128-column block (ld % 4 == 0, 16-byte aligned).
__global__ void __launch_bounds__(256) copy_upper_blocks_kernel(const float* __restrict__ src, int64_t lds,
                                                                float* __restrict__ dst, int64_t ldd, int64_t C) {
  const int64_t r = blockIdx.y;
  const int64_t c_begin = (r / 128) * 128;
  for (int64_t c = c_begin + ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; c < C; c += (int64_t)gridDim.x * blockDim.x * 4)
    *reinterpret_cast<float4*>(dst + r * ldd + c) = __ldg(reinterpret_cast<const float4*>(src + r * lds + c));
}
}  // namespace mq

extern "C" size_t mq_quantize_layer_workspace_bytes(int n_tied, int64_t R, int64_t C, int math, int split_hinv,
                                                    int split_sweep) {
  using namespace mq;
  if (n_tied <= 0 || R <= 0 || C <= 0) return 0;
  math &= ~MQ_MATH_COMPACT;
  size_t a = factor_workspace_bytes(C, math, split_hinv);            // factorisation: the planes of a super-panel
  size_t b = sweep_workspace_bytes(R, C, math, split_sweep);
  return layer_fixed_bytes(n_tied, R, C) + (a > b ? a : b);
}

extern "C" int mq_quantize_layer(const void* const* Wsrc, int w_dtype, int n_tied, int64_t R, int64_t C, float* H,
                                 int64_t ldh, int64_t group, int bits, float rel_damp, uint8_t* const* codes,
                                 int32_t* const* packed, float* const* scale_out, void* const* dequantized, mq_layer_flags* flags, int math,
                                 int split_hinv, int split_sweep, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace mq;
  MQ_REQUIRE(Wsrc && codes && scale_out && H && flags, MQ_ERR_ARGUMENT, "mq_quantize_layer: null pointer");
  MQ_REQUIRE(n_tied >= 1 && n_tied <= 8, MQ_ERR_ARGUMENT, "mq_quantize_layer: n_tied=%d", n_tied);
  MQ_REQUIRE(R > 0 && C > 0 && ldh >= C, MQ_ERR_ARGUMENT, "mq_quantize_layer: bad shape R=%lld C=%lld ldh=%lld", (long long)R,
             (long long)C, (long long)ldh);
  MQ_REQUIRE(valid_dtype(w_dtype), MQ_ERR_ARGUMENT, "mq_quantize_layer: bad dtype %d", w_dtype);
  MQ_REQUIRE(group > 0 && C % group == 0, MQ_ERR_ARGUMENT, "mq_quantize_layer: group %lld does not divide C=%lld",
             (long long)group, (long long)C);
  MQ_REQUIRE(bits >= 2 && bits <= 8, MQ_ERR_ARGUMENT, "mq_quantize_layer: bits=%d", bits);
  MQ_REQUIRE(C % 8 == 0, MQ_ERR_UNSUPPORTED, "mq_quantize_layer: C=%lld must be a multiple of 8", (long long)C);
  MQ_REQUIRE(ldh % 4 == 0 && aligned(H, 16), MQ_ERR_ALIGNMENT, "mq_quantize_layer: H must be 16-byte aligned, ldh %% 4 == 0");
  for (int i = 0; i < n_tied; ++i) {
    MQ_REQUIRE(Wsrc[i] && codes[i] && scale_out[i], MQ_ERR_ARGUMENT, "mq_quantize_layer: null pointer for tied layer %d", i);
    MQ_REQUIRE(aligned(codes[i], 4), MQ_ERR_ALIGNMENT, "mq_quantize_layer: codes must be 4-byte aligned");
    MQ_REQUIRE(!packed || (packed[i] && bits == 4 && aligned(packed[i], 4)), MQ_ERR_UNSUPPORTED,
               "mq_quantize_layer: packed words need bits == 4 and a 4-byte aligned buffer per layer");
  }
  const int sweep_math = math;   // the factorisation and the sweep honour MQ_MATH_COMPACT
  math &= ~MQ_MATH_COMPACT;
  MQ_REQUIRE(math == MQ_MATH_FP32 || math == MQ_MATH_TENSOR, MQ_ERR_ARGUMENT, "mq_quantize_layer: bad math %d", sweep_math);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Workspace ws(workspace, workspace_bytes);
  float* U = ws.take<float>((size_t)C * C);
  float* diag = ws.take<float>(C);
  float* Wf[8];
  float* Wo[8];
  for (int i = 0; i < n_tied; ++i) {
    Wf[i] = ws.take<float>((size_t)R * C);
    Wo[i] = ws.take<float>((size_t)R * C);
  }
  void* prep = ws.take<char>(mq_hessian_prepare_workspace_bytes(C));
  MQ_REQUIRE(U && diag && Wf[n_tied - 1] && Wo[n_tied - 1] && prep, MQ_ERR_WORKSPACE,
             "mq_quantize_layer: workspace of %zu bytes is too small", workspace_bytes);

  // W.clone().float()                                           src/gptq.py:149
  for (int i = 0; i < n_tied; ++i) MQ_TRY(launch_to_fp32(Wsrc[i], w_dtype, Wf[i], R * C, st));
  // pre-step + masking + damping, driven by the first layer's weight: the handle that owns H.
  // A tied handle meets an H that is already regularised and changes neither H nor its own
  // weight (src/gptq.py:129-136, 227).                          src/gptq.py:140-152, 224-234
  MQ_TRY(mq_hessian_prepare(H, C, ldh, Wf[0], R, C, rel_damp, flags, prep, mq_hessian_prepare_workspace_bytes(C), st));
  // grid                                                        src/quant_utils.py:75-101
  for (int i = 0; i < n_tied; ++i) MQ_TRY(mq_absmax_scales(Wf[i], R, C, C, group, bits, w_dtype, scale_out[i], st));
  // Factor a copy (the caller's H keeps the damped Hessian, which the reference leaves in
  // handle.H, quant.py:314-316).  Only the unit factor Utilde = T diag(T)^-1 of H = T T^T is
  // built: the sweep below runs in its inverse-free form, so the triangular inverse that
  // src/gptq.py:236-242 needs (and mq_hinv_upper provides) is never computed here.
  // With tensor math only the diagonal blocks of the factor are scaled by 1/diag(T) (the sweep
  // tiles read them); the blocks above are divided where they are split into planes.
  const bool unscaled = math == MQ_MATH_TENSOR;
  // The factorisation, the sweep tiles and the lazy updates read nothing below the diagonal
  // 128-blocks, so that half is neither copied nor zeroed.
  copy_upper_blocks_kernel<<<dim3(8, (unsigned)C), 256, 0, st>>>(H, ldh, U, C, C);
  MQ_LAUNCH_CHECK();
  {
    Workspace sub(ws.base + ws.used, ws.size - ws.used);
    MQ_TRY(chol_unit_factor(U, C, C, diag, sweep_math, split_hinv, flags, sub, st, true, unscaled));
  }
  // sweep                                                       src/gptq_loop.py:141-148
  for (int i = 0; i < n_tied; ++i) {
    MQ_CUDA(cudaMemcpyAsync(Wo[i], Wf[i], (size_t)R * C * sizeof(float), cudaMemcpyDeviceToDevice, st));
    Workspace sub(ws.base + ws.used, ws.size - ws.used);
    MQ_TRY(gptq_sweep(Wf[i], R, C, C, U, C, scale_out[i], nullptr, group, C / group, 1, bits, w_dtype, codes[i],
                      dequantized ? dequantized[i] : nullptr, Wo[i], C, sweep_math, split_sweep, sub, st, unscaled ? diag : nullptr,
                      packed ? packed[i] : nullptr));
  }
  return MQ_OK;
}
