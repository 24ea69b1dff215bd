// The Hessian-weighted error metric of the quantization loop,
//   get_relative_mse_error(q, w, H) = mean((q-w) H o (q-w)) / (mean(w H o w) + 1e-6)
// (src/quant_utils.py:259-264, called at quant.py:314-316 after every layer when errors are
// logged).  One quadratic form  sum_{r,c} (A H)[r,c] A[r,c]  per call: the product A H goes
// through the same contraction engine as the rest of the path (tcgen05 on split planes or fp32
// FMAs), the Hadamard product and the sum are one pass with fp64 accumulation.
#include "engine.cuh"

namespace mq {

__global__ void __launch_bounds__(256) dot_reduce_kernel(const float* __restrict__ T, int64_t ldt, const float* __restrict__ A,
                                                         int64_t lda, int64_t R, int64_t C, double* __restrict__ out) {
  double acc = 0.0;
  const int64_t n = R * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / C, c = i - r * C;
    acc += (double)T[r * ldt + c] * (double)A[r * lda + c];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  __shared__ double part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int w = 0; w < 8; ++w) s += part[w];
    atomicAdd(out, s);
  }
}

}  // namespace mq

extern "C" size_t mq_quadratic_form_workspace_bytes(int64_t R, int64_t C, int math, int split) {
  using namespace mq;
  if (R <= 0 || C <= 0) return 0;
  return align_up((size_t)R * C * sizeof(float), 256) + engine_workspace_bytes(R, C, C, math, split);
}

extern "C" int mq_quadratic_form(const float* A, int64_t R, int64_t C, int64_t lda, const float* H, int64_t ldh, double* out,
                                 int math, int split, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace mq;
  MQ_REQUIRE(A && H && out, MQ_ERR_ARGUMENT, "mq_quadratic_form: null pointer");
  MQ_REQUIRE(R > 0 && C > 0 && lda >= C && ldh >= C, MQ_ERR_ARGUMENT, "mq_quadratic_form: bad shape R=%lld C=%lld lda=%lld ldh=%lld",
             (long long)R, (long long)C, (long long)lda, (long long)ldh);
  MQ_REQUIRE(math == MQ_MATH_FP32 || math == MQ_MATH_TENSOR, MQ_ERR_ARGUMENT, "mq_quadratic_form: bad math %d", math);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Workspace ws(workspace, workspace_bytes);
  float* T = ws.take<float>((size_t)R * C);
  MQ_REQUIRE(T, MQ_ERR_WORKSPACE, "mq_quadratic_form: workspace of %zu bytes is too small", workspace_bytes);
  GemmDesc g;
  g.A = A; g.a_rs = lda; g.a_cs = 1;
  g.B = H; g.b_rs = ldh; g.b_cs = 1;
  g.C = T; g.ldc = C;
  g.M = (int)R; g.N = (int)C; g.K = (int)C;
  g.alpha = 1.0f; g.beta = 0.0f;
  Engine eng(math, split, ws, st);
  MQ_TRY(eng.gemm(g));
  MQ_CUDA(cudaMemsetAsync(out, 0, sizeof(double), st));
  const int64_t blocks = ceil_div(R * C, 256 * 8);
  dot_reduce_kernel<<<(unsigned)(blocks < 148 * 8 ? (blocks < 1 ? 1 : blocks) : 148 * 8), 256, 0, st>>>(T, C, A, lda, R, C, out);
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}
