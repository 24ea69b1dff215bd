// Dense-contraction interface shared by the Hessian, the factorisation and the
// lazy block update.  Two implementations sit behind it: fp32 FMAs on the CUDA
// cores (gemm_simt.cu) and tcgen05 tensor cores on bf16 planes (umma_gemm.cu).
#pragma once

#include "common.cuh"

namespace mq {

// C[m,n] = alpha * sum_k A[m,k] B[k,n] + beta * C[m,n], fp32 output.
// A[m,k] lives at A[m*a_rs + k*a_cs], B[k,n] at B[k*b_rs + n*b_cs], C[m,n] at C[m*ldc + n].
struct GemmDesc {
  const void* A = nullptr;
  int64_t a_rs = 0, a_cs = 0;
  const void* B = nullptr;
  int64_t b_rs = 0, b_cs = 0;
  float* C = nullptr;
  int64_t ldc = 0;
  int M = 0, N = 0, K = 0;
  float alpha = 1.0f, beta = 0.0f;
  // Structure that lets whole tiles or k-ranges be skipped:
  int upper_tiles_only = 0;  // skip output tiles that lie entirely below the diagonal
  int mirror_to_lower = 0;   // with upper_tiles_only on a symmetric result: also write C[n,m] = C[m,n] (tensor path)
  int a_upper = 0;           // A is upper triangular (A[m,k] == 0 for k < m): k starts at the tile's first row
  int b_upper = 0;           // B is upper triangular (B[k,n] == 0 for k > n): k stops at the tile's last column
  // Batched form: operand b lives at base + b * stride (elements of the operand type).
  int batch = 1;
  int64_t a_bs = 0, b_bs = 0, c_bs = 0;
  // Ragged last batch: batch b sees N_b = min(N, n_total - b * n_step) columns and, when
  // k_follows_n is set, K_b = N_b as well (the D^-1 factor of a triangular merge).
  int n_total = 0, n_step = 0, k_follows_n = 0;
  // Tensor path, beta == 1, K > k_round > 0 (a multiple of 64): the partial sums of every k_round
  // columns of k are added to C one after the other in round-to-nearest fp32, as separate
  // updates of depth k_round would, instead of meeting inside the tensor core's accumulator.
  int k_round = 0;
  // Tensor path, rank-<=128 updates: the caller runs several layers at once (MQ_MATH_COMPACT), so
  // a CTA walks a whole row of output tiles: half to a third of the CTAs, each a little longer.
  int compact = 0;
};

// fp32 CUDA-core implementation; in_dtype is the element type of A and B.
int gemm_simt(const GemmDesc& d, int in_dtype, cudaStream_t st);

// Work of one GEMM launch: algorithmic flop (2 per multiply-add on the tiles and k-ranges
// that the structure flags keep, unpadded) and issued flop (padded tiles x products).
void gemm_work(const GemmDesc& d, int k_granule, double* algorithmic, double* issued, int products);

// Copies the strict upper triangle of a square matrix onto its lower triangle.
int mirror_upper_to_lower(float* H, int64_t C, int64_t ldh, cudaStream_t st);

}  // namespace mq
