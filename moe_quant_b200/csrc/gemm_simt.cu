// fp32 CUDA-core GEMM with arbitrary operand strides, triangular tile skipping
// and a batched form.  This is the MQ_MATH_FP32 arithmetic: plain fp32 FMAs, the
// same number format as the reference's TF32-off cuBLAS calls
// (src/gptq.py:13-14, 103; src/gptq_loop.py:148).  128x128x8 tiles, 8x8 outputs
// per thread, double-buffered shared memory.
#include "gemm.cuh"
#include "profile.cuh"

namespace mq {

namespace {

constexpr int BM = 128, BN = 128, BK = 8, PAD = 4, THREADS = 256;

template <typename T, bool A_M_CONTIG, bool B_N_CONTIG>
__global__ void __launch_bounds__(THREADS) gemm_simt_kernel(GemmDesc d) {
  const int b = blockIdx.z;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  int N = d.N, K = d.K;
  if (d.n_step) {
    int left = d.n_total - b * d.n_step;
    N = N < left ? N : left;
    if (d.k_follows_n) K = N;
  }
  if (N <= 0 || n0 >= N || m0 >= d.M) return;
  if (d.upper_tiles_only && n0 + BN <= m0) return;
  const T* __restrict__ A = static_cast<const T*>(d.A) + (int64_t)b * d.a_bs;
  const T* __restrict__ B = static_cast<const T*>(d.B) + (int64_t)b * d.b_bs;
  float* __restrict__ C = d.C + (int64_t)b * d.c_bs;
  const int M = d.M;
  const int k_lo = d.a_upper ? m0 : 0;  // m0 is a multiple of BK
  int k_hi = K;
  if (d.b_upper && n0 + BN < k_hi) k_hi = n0 + BN;

  __shared__ __align__(16) float As[2][BK][BM + PAD];
  __shared__ __align__(16) float Bs[2][BK][BN + PAD];

  const int t = threadIdx.x;
  const int tx = t & 15, ty = t >> 4;

  float ra[4], rb[4];
  auto load_tiles = [&](int k0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int m, k;
      if (A_M_CONTIG) { m = t & 127; k = (t >> 7) + 2 * i; } else { k = t & 7; m = (t >> 3) + 32 * i; }
      int gm = m0 + m, gk = k0 + k;
      ra[i] = (gm < M && gk < k_hi) ? to_float(A[(int64_t)gm * d.a_rs + (int64_t)gk * d.a_cs]) : 0.0f;
      int n;
      if (B_N_CONTIG) { n = t & 127; k = (t >> 7) + 2 * i; } else { k = t & 7; n = (t >> 3) + 32 * i; }
      int gn = n0 + n;
      gk = k0 + k;
      rb[i] = (gn < N && gk < k_hi) ? to_float(B[(int64_t)gk * d.b_rs + (int64_t)gn * d.b_cs]) : 0.0f;
    }
  };
  auto store_tiles = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int m, k;
      if (A_M_CONTIG) { m = t & 127; k = (t >> 7) + 2 * i; } else { k = t & 7; m = (t >> 3) + 32 * i; }
      As[buf][k][m] = ra[i];
      int n;
      if (B_N_CONTIG) { n = t & 127; k = (t >> 7) + 2 * i; } else { k = t & 7; n = (t >> 3) + 32 * i; }
      Bs[buf][k][n] = rb[i];
    }
  };

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

  if (k_lo < k_hi) {
    load_tiles(k_lo);
    store_tiles(0);
    __syncthreads();
    int buf = 0;
    for (int k0 = k_lo; k0 < k_hi; k0 += BK) {
      const bool more = k0 + BK < k_hi;
      if (more) load_tiles(k0 + BK);
#pragma unroll
      for (int k = 0; k < BK; ++k) {
        float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
        float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
        float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
        float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
        float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
      }
      if (more) {
        store_tiles(buf ^ 1);
        __syncthreads();
        buf ^= 1;
      }
    }
  }

  const float alpha = d.alpha, beta = d.beta;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (gm >= M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int gn = n0 + h * 64 + tx * 4;
      float* p = C + (int64_t)gm * d.ldc + gn;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (gn + j < N) {
          float v = alpha * acc[i][h * 4 + j];
          if (beta != 0.0f) v = fmaf(beta, p[j], v);
          p[j] = v;
        }
      }
    }
  }
}

template <typename T>
int launch(const GemmDesc& d, cudaStream_t st) {
  dim3 grid((unsigned)ceil_div(d.N, BN), (unsigned)ceil_div(d.M, BM), (unsigned)d.batch);
  bool am = d.a_rs == 1, bn = d.b_cs == 1;
  if (am && bn)
    gemm_simt_kernel<T, true, true><<<grid, THREADS, 0, st>>>(d);
  else if (am && !bn)
    gemm_simt_kernel<T, true, false><<<grid, THREADS, 0, st>>>(d);
  else if (!am && bn)
    gemm_simt_kernel<T, false, true><<<grid, THREADS, 0, st>>>(d);
  else
    gemm_simt_kernel<T, false, false><<<grid, THREADS, 0, st>>>(d);
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}

__global__ void __launch_bounds__(256) mirror_kernel(float* __restrict__ H, int64_t C, int64_t ldh) {
  // 32x32 tiles strictly above or on the diagonal are transposed through shared memory
  // onto their mirror image; blockIdx.x >= blockIdx.y only.
  __shared__ float tile[32][33];
  int bx = blockIdx.x, by = blockIdx.y;
  if (bx < by) return;
  int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int i = ty; i < 32; i += 8) {
    int64_t r = (int64_t)by * 32 + i, c = (int64_t)bx * 32 + tx;
    tile[i][tx] = (r < C && c < C) ? H[r * ldh + c] : 0.0f;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    int64_t r = (int64_t)bx * 32 + i, c = (int64_t)by * 32 + tx;  // mirrored position
    if (r < C && c < C && r > c) H[r * ldh + c] = tile[tx][i];
  }
}

}  // namespace

void gemm_work(const GemmDesc& d, int k_granule, double* algorithmic, double* issued, int products) {
  double alg = 0.0, iss = 0.0;
  for (int b = 0; b < d.batch; ++b) {
    int N = d.N, K = d.K;
    if (d.n_step) {
      int left = d.n_total - b * d.n_step;
      N = N < left ? N : left;
      if (d.k_follows_n) K = N;
    }
    if (N <= 0) continue;
    for (int m0 = 0; m0 < d.M; m0 += 128) {
      for (int n0 = 0; n0 < N; n0 += 128) {
        if (d.upper_tiles_only && n0 + 128 <= m0) continue;
        int k_lo = d.a_upper ? m0 : 0;
        int k_hi = K;
        if (d.b_upper && n0 + 128 < k_hi) k_hi = n0 + 128;
        if (k_hi <= k_lo) continue;
        int rows = d.M - m0 < 128 ? d.M - m0 : 128, cols = N - n0 < 128 ? N - n0 : 128;
        alg += 2.0 * rows * cols * (k_hi - k_lo);
        int kp = (k_hi - k_lo + k_granule - 1) / k_granule * k_granule;
        iss += 2.0 * 128 * 128 * kp * products;
      }
    }
  }
  *algorithmic = alg;
  *issued = iss;
}

int gemm_simt(const GemmDesc& d, int in_dtype, cudaStream_t st) {
  if (d.M <= 0 || d.N <= 0 || d.batch <= 0) return MQ_OK;
  double flop_alg = 0.0, flop_issued = 0.0;
  if (g_profile_on) gemm_work(d, 8, &flop_alg, &flop_issued, 1);
  ProfScope prof(PROF_SIMT_GEMM, flop_alg, flop_issued, st);
  switch (in_dtype) {
    case MQ_F32: return launch<float>(d, st);
    case MQ_BF16: return launch<__nv_bfloat16>(d, st);
    case MQ_F16: return launch<__half>(d, st);
  }
  set_error("gemm_simt: bad dtype %d", in_dtype);
  return MQ_ERR_ARGUMENT;
}

int mirror_upper_to_lower(float* H, int64_t C, int64_t ldh, cudaStream_t st) {
  dim3 grid((unsigned)ceil_div(C, 32), (unsigned)ceil_div(C, 32));
  mirror_kernel<<<grid, 256, 0, st>>>(H, C, ldh);
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}

}  // namespace mq
