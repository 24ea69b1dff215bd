// Uhat = row-normalised upper Cholesky factor of H^-1, computed without ever
// forming H^-1:
//
//   H = T T^T with T upper triangular (a Cholesky factorisation that starts at the
//   bottom-right corner), so chol_upper(H^-1) = T^-1 and, after dividing each row
//   by its diagonal,  Uhat = diag(T) T^-1 = (T diag(T)^-1)^-1.
//
// One factorisation (C^3/3 flop) and one unit-triangular inverse (C^3/3) replace
// the reference's potrf + potri + potrf (src/linalg_utils.py:12,
// src/gptq.py:237-242; about 4C^3/3 flop).
//
// Blocked right-looking factorisation with 128-wide panels processed from the last
// panel to the first:
//   1. chol_diag_rev_kernel  : the 128x128 diagonal block, one CTA, register tiled;
//   2. trsm_rows_kernel      : the panel above it, one warp per row, substitution
//                              against the diagonal block staged in shared memory;
//   3. GEMMs (GemmDesc)      : trailing update of the upper triangle; on the tensor path in two
//                              levels (the rest of the panel's 512-column super-panel at once,
//                              everything in front of the super-panel once per super-panel with
//                              all 512 columns in the contraction).
// The inverse is built by inverting the 128x128 diagonal blocks (same substitution
// kernel on identity rows) and then merging neighbouring blocks pairwise,
//   inv([A B; 0 D]) = [A^-1, -A^-1 B D^-1; 0, D^-1],
// log2(C/128) levels of two batched GEMMs each.
#include "gemm.cuh"
#include "engine.cuh"
#include "profile.cuh"

namespace mq {

namespace {

constexpr int NB = 128;  // panel width
constexpr int SUPER_PANELS = 4;               // panels whose far update is applied together
constexpr int SUPER_NB = SUPER_PANELS * NB;   // 512

// ------------------------------------------------------------------ diagonal block
// D (nb x nb, upper triangle valid) -> T_d upper with D = T_d T_d^T, one CTA of 512 threads.
// The block lives in shared memory.  The 128 pivots are taken 8 at a time (a "leaf", columns
// 8kt..8kt+7, kt = 15 first).  One warp's instruction stream runs at a fraction of an instruction
// per cycle here (every step depends on the one before), so a leaf is arranged to put as few
// instructions as possible in any one stream:
//   a. thread r < 8kt + 8 takes ROW r of the column strip: it factors its own copy of the 8x8
//      leaf in registers (the same arithmetic in every thread, no communication inside the chain
//      of 8 pivots) and solves its own row against it; the row's eight results are final: they go
//      to global memory at once and, transposed, to the panel buffer;
//   b. every element on or above the diagonal tiles in front of the strip takes its rank-8 update
//      from the panel buffer.  The region shrinks with every leaf, so its 4x4 micro-tiles are dealt
//      out to all 512 threads anew each time (with the tiles in registers of fixed owners, four
//      fifths of the lanes idled through this phase, which the FMA pipe of the one SM bounds).
constexpr int PAN_LD = NB + 4;
constexpr int DIAG_THREADS = 512;
constexpr int DIAG_LD = NB + 4;   // row stride of the block in shared memory (16-byte aligned rows)
constexpr size_t kDiagSmem = (size_t)NB * DIAG_LD * sizeof(float);

__global__ void __launch_bounds__(DIAG_THREADS) chol_diag_rev_kernel(float* __restrict__ blk, int64_t ld, int nb,
                                                                     int k_global, mq_layer_flags* flags) {
  extern __shared__ __align__(16) float Ms[];         // [NB][DIAG_LD]: the block, tiles on and above the diagonal
  __shared__ __align__(16) float pan[8][PAN_LD];      // pan[kk][row]: column 8kt+kk of the solved strip
  chain_wait();
  chain_release();
  const int t = threadIdx.x;
  // A whole, 16-byte aligned block moves as float4; rows and columns past nb read as the identity.
  const bool vec = nb == NB && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(blk) & 15) == 0;
  for (int idx = t; idx < NB * NB / 4; idx += DIAG_THREADS) {
    const int r = idx >> 5, c4 = (idx & 31) * 4;
    if ((c4 >> 3) < (r >> 3)) continue;               // tiles below the diagonal are never read
    float4 v;
    if (vec) {
      v = *reinterpret_cast<const float4*>(blk + (int64_t)r * ld + c4);
    } else {
      float e[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) e[q] = (r < nb && c4 + q < nb) ? blk[(int64_t)r * ld + c4 + q] : (r == c4 + q ? 1.0f : 0.0f);
      v = make_float4(e[0], e[1], e[2], e[3]);
    }
    *reinterpret_cast<float4*>(&Ms[r * DIAG_LD + c4]) = v;
  }
  __syncthreads();
  for (int kt = 15; kt >= 0; --kt) {
    // ---- a. one row of the strip per thread
    const int row = t;
    if (row < kt * 8 + 8) {
      float L[8][8];   // L[i][j] = leaf element (row 8kt+i, column 8kt+j), upper triangle
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 lo = *reinterpret_cast<const float4*>(&Ms[(kt * 8 + i) * DIAG_LD + kt * 8]);
        const float4 hi = *reinterpret_cast<const float4*>(&Ms[(kt * 8 + i) * DIAG_LD + kt * 8 + 4]);
        L[i][0] = lo.x; L[i][1] = lo.y; L[i][2] = lo.z; L[i][3] = lo.w;
        L[i][4] = hi.x; L[i][5] = hi.y; L[i][6] = hi.z; L[i][7] = hi.w;
      }
      float x[8];
      {
        const float4 lo = *reinterpret_cast<const float4*>(&Ms[row * DIAG_LD + kt * 8]);
        const float4 hi = *reinterpret_cast<const float4*>(&Ms[row * DIAG_LD + kt * 8 + 4]);
        x[0] = lo.x; x[1] = lo.y; x[2] = lo.z; x[3] = lo.w; x[4] = hi.x; x[5] = hi.y; x[6] = hi.z; x[7] = hi.w;
      }
      // The 8 pivots are one straight line of code (no branch), so that the scheduler can put
      // the row arithmetic of pivot kk into the latency of pivot kk-1's rsqrt chain.  The rows
      // of the leaf itself run the row arithmetic too; that copy is discarded below.
      int fail = 0;
#pragma unroll
      for (int kk = 7; kk >= 0; --kk) {
        float d = L[kk][kk];
        const bool bad = !(d > 0.0f);  // also catches NaN
        fail = (bad && fail == 0) ? kk + 1 : fail;
        d = bad ? 1.0f : d;
        float r;                       // d is a positive, normal pivot (or 1): the hardware approximation, refined below
        asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
        r = r * fmaf(-0.5f * d * r, r, 1.5f);  // one Newton step: r = 1/sqrt(d) to about 1 ulp
        L[kk][kk] = d * r;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (i < kk) L[i][kk] *= r;
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (i <= j && j < kk) L[i][j] = fmaf(-L[i][kk], L[j][kk], L[i][j]);
        // this row above the leaf: p_kk = x_kk / T[kk][kk]; x_j -= p_kk T[j][kk]  (j < kk)
        const float pv = x[kk] * r;
        x[kk] = pv;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < kk) x[j] = fmaf(-pv, L[j][kk], x[j]);
      }
      const int li = row - kt * 8;   // >= 0: a row of the leaf, which gets the factor instead
      if (li >= 0) {
        if (li == 0 && fail != 0 && kt * 8 + fail - 1 < nb) atomicCAS(&flags->not_positive, 0, k_global + kt * 8 + fail);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          float v = 0.0f;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (i == li && i <= kk) v = L[i][kk];
          x[kk] = v;
        }
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) pan[kk][row] = x[kk];
      // the strip is final
      if (vec) {
        *reinterpret_cast<float4*>(blk + (int64_t)row * ld + kt * 8) = make_float4(x[0], x[1], x[2], x[3]);
        *reinterpret_cast<float4*>(blk + (int64_t)row * ld + kt * 8 + 4) = make_float4(x[4], x[5], x[6], x[7]);
      } else if (row < nb) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          if (kt * 8 + kk < nb) blk[(int64_t)row * ld + kt * 8 + kk] = x[kk];
      }
    } else if (row < NB) {
      // below the leaf: zeros
      if (vec) {
        *reinterpret_cast<float4*>(blk + (int64_t)row * ld + kt * 8) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(blk + (int64_t)row * ld + kt * 8 + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
      } else if (row < nb) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          if (kt * 8 + kk < nb) blk[(int64_t)row * ld + kt * 8 + kk] = 0.0f;
      }
    }
    __syncthreads();
    // ---- b. rank-8 update of what lies in front of the strip: rows and columns below 8kt, 4x4
    // micro-tiles on and above the diagonal 8x8 tiles.  n micro-rows (even); rows i and n-1-i
    // together hold n + 1 micro-tiles on or right of the diagonal, which makes the triangle a
    // rectangle of n/2 x (n + 1) items.  (A micro-tile left of the diagonal micro-tile of its
    // row but inside a diagonal 8x8 tile is never read: it is skipped with the rest.)
    const int n = 2 * kt;
    const int items = (n >> 1) * (n + 1);
    for (int m = t; m < items; m += DIAG_THREADS) {
      const int i = m / (n + 1), jj = m - i * (n + 1);
      int mi, mj;
      if (jj < n - i) { mi = i; mj = i + jj; }
      else { mi = n - 1 - i; mj = mi + (jj - (n - i)); }
      const int r0 = 4 * mi, c0 = 4 * mj;
      float c[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float4 v = *reinterpret_cast<const float4*>(&Ms[(r0 + a) * DIAG_LD + c0]);
        c[a][0] = v.x; c[a][1] = v.y; c[a][2] = v.z; c[a][3] = v.w;
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const float4 pi4 = *reinterpret_cast<const float4*>(&pan[kk][r0]);
        const float4 pj4 = *reinterpret_cast<const float4*>(&pan[kk][c0]);
        const float pi[4] = {pi4.x, pi4.y, pi4.z, pi4.w};
        // two columns per instruction (packed fp32 FMA: each half is an ordinary fma.rn)
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const float2 npi = make_float2(-pi[a], -pi[a]);
          const float2 q01 = __ffma2_rn(npi, make_float2(pj4.x, pj4.y), make_float2(c[a][0], c[a][1]));
          const float2 q23 = __ffma2_rn(npi, make_float2(pj4.z, pj4.w), make_float2(c[a][2], c[a][3]));
          c[a][0] = q01.x; c[a][1] = q01.y; c[a][2] = q23.x; c[a][3] = q23.y;
        }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a)
        *reinterpret_cast<float4*>(&Ms[(r0 + a) * DIAG_LD + c0]) = make_float4(c[a][0], c[a][1], c[a][2], c[a][3]);
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------ substitution
// Solves P T^T = A row by row, T the (nb x nb) upper-triangular block at `tblk`:
//   for k = nb-1 .. 0:  p_k = a_k / T[k,k];  a_j -= p_k T[j,k]  (j < k).
// One warp per row; lane l holds columns 4l..4l+3.  T is staged transposed in shared
// memory so that a lane reads the four T[j,k] it needs as one float4.
// IDENTITY: the right-hand side is I and the result is stored transposed, which
// yields T^-1 (upper triangular) in `rows`.
constexpr int TT_LD = NB + 4;

template <bool IDENTITY>
__global__ void __launch_bounds__(256) trsm_rows_kernel(const float* __restrict__ tblk, int64_t ldt, int64_t t_bs,
                                                        float* __restrict__ rows, int64_t ldr, int64_t r_bs,
                                                        int nrows, int nb_full, int n_total,
                                                        uint16_t* __restrict__ planes, int64_t plane_stride, int n_planes,
                                                        int plane_ld) {
  extern __shared__ __align__(16) float smem[];
  float* TT = smem;                // [NB][TT_LD], TT[k][j] = T[j][k] for j < k, else 0
  float* dg = smem + NB * TT_LD;   // [NB] diagonal of T
  float* rdg = dg + NB;            // [NB] its reciprocal
  const int b = blockIdx.y;
  int nb = nb_full;
  if (n_total > 0) {  // batched over diagonal blocks: the last one may be narrower
    int left = n_total - b * nb_full;
    nb = left < nb_full ? left : nb_full;
    if (IDENTITY) nrows = nb;
  }
  tblk += (int64_t)b * t_bs;
  rows += (int64_t)b * r_bs;
  // Four rows per warp at a time share each shared-memory read of TT and give the scheduler four
  // independent shuffle/FMA chains.
  constexpr int ROWS = 4;
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int r_first = ROWS * (blockIdx.x * warps_per_block + (threadIdx.x >> 5));
  float a[ROWS][4];
  // The rows of the panel were final before the diagonal block in front of this launch was
  // factored (that kernel writes only the block), so the first rows are fetched before this grid
  // waits for it; the block itself is staged after the wait.
  if (!IDENTITY) {
#pragma unroll
    for (int h = 0; h < ROWS; ++h) {
      const int r = r_first + h;
      if (r < nrows && lane * 4 < nb) {
        float4 v = *reinterpret_cast<const float4*>(rows + (int64_t)r * ldr + lane * 4);
        a[h][0] = v.x; a[h][1] = v.y; a[h][2] = v.z; a[h][3] = v.w;
      } else {
        a[h][0] = a[h][1] = a[h][2] = a[h][3] = 0.0f;
      }
    }
  }
  chain_wait();
  chain_release();
  {
    // Up to 16 independent float4 loads per thread plus the diagonal are issued before any is used
    // (one memory latency for the block); quads that lie below the diagonal are zeros in the
    // staged form and are not loaded.  float4 index: row j = idx % 128, columns
    // k4..k4+3; consecutive threads take consecutive rows so that the transposed shared-memory
    // stores hit 32 different banks.
    float4 v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int j = idx & 127, k4 = (idx >> 7) * 4;
      v[i] = (j < nb && k4 < nb && k4 + 3 > j) ? __ldg(reinterpret_cast<const float4*>(tblk + (int64_t)j * ldt + k4))
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (threadIdx.x < NB) {
      const int k = threadIdx.x;
      const float d = k < nb ? __ldg(tblk + (int64_t)k * ldt + k) : 1.0f;
      dg[k] = d;
      rdg[k] = 1.0f / d;
    }
    __syncthreads();
    // The block is staged with every column already divided by its diagonal entry
    // (TT[k][j] = T[j][k] / T[k][k], zero for j >= k), so a substitution step is
    // a_j -= a_k * TT[k][j]: no division and no write-back of a_k inside the chain; the quotients
    // p_k = a_k / T[k][k] are formed once at the end.
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int j = idx & 127, k4 = (idx >> 7) * 4;
      const float4 r4 = *reinterpret_cast<const float4*>(&rdg[k4]);
      const float e[4] = {v[i].x * r4.x, v[i].y * r4.y, v[i].z * r4.z, v[i].w * r4.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) TT[(k4 + q) * TT_LD + j] = (j < k4 + q && k4 + q < nb) ? e[q] : 0.0f;
    }
  }
  __syncthreads();
  for (int r0 = r_first; r0 < nrows; r0 += ROWS * gridDim.x * warps_per_block) {
#pragma unroll
    for (int h = 0; h < ROWS; ++h) {
      const int r = r0 + h;
      if (IDENTITY) {
#pragma unroll
        for (int q = 0; q < 4; ++q) a[h][q] = (lane * 4 + q == r) ? 1.0f : 0.0f;
      } else if (r0 == r_first) {
        // fetched before the wait
      } else if (r < nrows && lane * 4 < nb) {
        float4 v = *reinterpret_cast<const float4*>(rows + (int64_t)r * ldr + lane * 4);
        a[h][0] = v.x; a[h][1] = v.y; a[h][2] = v.z; a[h][3] = v.w;
      } else {
        a[h][0] = a[h][1] = a[h][2] = a[h][3] = 0.0f;
      }
    }
    for (int kq = (nb >> 2) - 1; kq >= 0; --kq) {
#pragma unroll
      for (int kk = 3; kk >= 0; --kk) {
        const float4 tt = *reinterpret_cast<const float4*>(&TT[(kq * 4 + kk) * TT_LD + lane * 4]);
#pragma unroll
        for (int h = 0; h < ROWS; ++h) {
          const float ak = __shfl_sync(0xffffffffu, a[h][kk], kq);
          // packed fp32 FMA: two columns per instruction, each half an ordinary fma.rn
          const float2 nak = make_float2(-ak, -ak);
          const float2 lo = __ffma2_rn(nak, make_float2(tt.x, tt.y), make_float2(a[h][0], a[h][1]));
          const float2 hi = __ffma2_rn(nak, make_float2(tt.z, tt.w), make_float2(a[h][2], a[h][3]));
          a[h][0] = lo.x; a[h][1] = lo.y; a[h][2] = hi.x; a[h][3] = hi.y;
        }
      }
    }
    {
      const float4 d4 = *reinterpret_cast<const float4*>(&dg[lane * 4]);
      const float4 r4 = *reinterpret_cast<const float4*>(&rdg[lane * 4]);
      const float dd[4] = {d4.x, d4.y, d4.z, d4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
      for (int h = 0; h < ROWS; ++h)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          // a / d through the reciprocal and one correction step (the last stage of a correctly
          // rounded division)
          float pq = a[h][q] * rr[q];
          a[h][q] = fmaf(fmaf(-dd[q], pq, a[h][q]), rr[q], pq);
        }
    }
    if (lane * 4 < nb) {
#pragma unroll
      for (int h = 0; h < ROWS; ++h) {
        const int r = r0 + h;
        if (r >= nrows) continue;
        if (IDENTITY) {
          // result row r is column r of T^-1
#pragma unroll
          for (int q = 0; q < 4; ++q) rows[(int64_t)(lane * 4 + q) * ldr + r] = a[h][q];
        } else {
          *reinterpret_cast<float4*>(rows + (int64_t)r * ldr + lane * 4) = make_float4(a[h][0], a[h][1], a[h][2], a[h][3]);
        }
      }
    }
    if (!IDENTITY && planes) {
      // the trailing update reads this panel as bf16 planes (row, k = column inside the panel)
#pragma unroll
      for (int h = 0; h < ROWS; ++h) {
        const int r = r0 + h;
        if (r >= nrows) continue;
        uint16_t hi[4], mi[4], lo[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) split_bf16x3(lane * 4 < nb ? a[h][q] : 0.0f, hi[q], mi[q], lo[q]);
        uint16_t* dst = planes + (int64_t)r * plane_ld + lane * 4;   // `planes` already points at this panel's k window
        *reinterpret_cast<uint2*>(dst) = make_uint2((uint32_t)hi[0] | ((uint32_t)hi[1] << 16), (uint32_t)hi[2] | ((uint32_t)hi[3] << 16));
        if (n_planes > 1)
          *reinterpret_cast<uint2*>(dst + plane_stride) =
              make_uint2((uint32_t)mi[0] | ((uint32_t)mi[1] << 16), (uint32_t)mi[2] | ((uint32_t)mi[3] << 16));
        if (n_planes > 2)
          *reinterpret_cast<uint2*>(dst + 2 * plane_stride) =
              make_uint2((uint32_t)lo[0] | ((uint32_t)lo[1] << 16), (uint32_t)lo[2] | ((uint32_t)lo[3] << 16));
      }
    }
  }
}

// ------------------------------------------------------------------ small passes
__global__ void __launch_bounds__(256) extract_diag_kernel(const float* __restrict__ H, int64_t C, int64_t ld,
                                                           float* __restrict__ diag) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < C) diag[i] = H[i * ld + i];
}

// T -> T diag(T)^-1 on the upper triangle (unit diagonal), zeros below it.
// upper_only = 1: what lies entirely below the diagonal is left as it is instead of being zeroed
// (the layer path never reads it); = 2: in addition only the diagonal 128-blocks are scaled (the
// sweep tiles read those; the blocks above are divided by whoever splits them into planes).
__device__ __forceinline__ void scale_quad(float* __restrict__ H, int64_t ld, const float* __restrict__ diag, int64_t r,
                                           int64_t c) {
  // four columns c..c+3 of row r; what lies entirely below the diagonal is written without being read
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c + 3 >= r) {
    const float4 v = *reinterpret_cast<const float4*>(H + r * ld + c);
    const float4 d = __ldg(reinterpret_cast<const float4*>(diag + c));
    o.x = (c + 0 > r) ? v.x / d.x : (c + 0 == r ? 1.0f : 0.0f);
    o.y = (c + 1 > r) ? v.y / d.y : (c + 1 == r ? 1.0f : 0.0f);
    o.z = (c + 2 > r) ? v.z / d.z : (c + 2 == r ? 1.0f : 0.0f);
    o.w = (c + 3 > r) ? v.w / d.w : (c + 3 == r ? 1.0f : 0.0f);
  }
  *reinterpret_cast<float4*>(H + r * ld + c) = o;
}

__global__ void __launch_bounds__(256) scale_columns_kernel(float* __restrict__ H, int64_t C, int64_t ld,
                                                            const float* __restrict__ diag, int upper_only) {
  const int64_t r = blockIdx.y;
  if ((C & 3) == 0 && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(H) & 15) == 0) {
    if (upper_only == 2) {  // launched with one block of 32 threads per row: the row's diagonal block
      const int64_t c = (r / NB) * NB + threadIdx.x * 4;
      if (blockIdx.x == 0 && threadIdx.x < NB / 4 && c < C && c + 3 >= r) scale_quad(H, ld, diag, r, c);
      return;
    }
    for (int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; c < C; c += (int64_t)gridDim.x * blockDim.x * 4) {
      if (upper_only && c + 3 < r) continue;
      scale_quad(H, ld, diag, r, c);
    }
    return;
  }
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < C; c += (int64_t)gridDim.x * blockDim.x) {
    if (upper_only == 2 && (c < (r / NB) * NB || c >= (r / NB + 1) * NB)) continue;
    float v = H[r * ld + c];
    H[r * ld + c] = (c > r) ? v / diag[c] : (c == r ? 1.0f : 0.0f);
  }
}

__global__ void __launch_bounds__(256) identity_if_failed_kernel(float* __restrict__ U, int64_t C, int64_t ld,
                                                                 const mq_layer_flags* flags, float* __restrict__ diag) {
  if (flags->not_positive == 0) return;
  // with the identity as factor its column scaling is 1 as well (a caller that was handed the
  // unscaled factor divides by it)
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < C; i += (int64_t)gridDim.x * blockDim.x) diag[i] = 1.0f;
  int64_t n = C * C;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / C, c = i - r * C;
    U[r * ld + c] = (r == c) ? 1.0f : 0.0f;
  }
}

constexpr size_t kTrsmSmem = (size_t)(NB * TT_LD + 2 * NB) * sizeof(float);

int configure_once() {
  static bool done[64] = {};
  int dev = 0;
  MQ_CUDA(cudaGetDevice(&dev));
  if (!done[dev & 63]) {
    MQ_CUDA(cudaFuncSetAttribute(chol_diag_rev_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDiagSmem));
    MQ_CUDA(cudaFuncSetAttribute(trsm_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTrsmSmem));
    MQ_CUDA(cudaFuncSetAttribute(trsm_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTrsmSmem));
    done[dev & 63] = true;
  }
  return MQ_OK;
}

}  // namespace

size_t factor_workspace_bytes(int64_t C, int math, int split) {
  return math == MQ_MATH_TENSOR ? plane_set_bytes(C, SUPER_NB, split) : 0;
}

size_t hinv_workspace_bytes(int64_t C, int math, int split) {
  size_t bytes = align_up((size_t)C * sizeof(float), 256);          // diag
  bytes += align_up((size_t)C * (size_t)C * sizeof(float), 256);    // merge scratch
  size_t a = engine_workspace_bytes(C, C, C, math, split), b = factor_workspace_bytes(C, math, split);
  bytes += a > b ? a : b;
  return bytes;
}

// H (damped, symmetric; upper triangle read) -> unit upper factor Utilde = T diag(T)^-1 in place,
// zeros below the diagonal (upper_only: the part below the diagonal blocks is neither read nor written;
// unscaled: only the diagonal blocks are scaled; above them T itself is left in place and the caller
// divides column c by diag[c] where it reads it).  diag (C floats, device) receives diag(T).  On a non-positive pivot
// flags->not_positive is set and the result is replaced by I.
int chol_unit_factor(float* H, int64_t C, int64_t ldh, float* diag, int math, int split, mq_layer_flags* flags,
                     Workspace& ws, cudaStream_t st, bool upper_only, bool unscaled) {
  MQ_TRY(configure_once());
  const int compact = (math & MQ_MATH_COMPACT) ? 1 : 0;   // the panel solves and the rank-128 strips look at it
  math &= ~MQ_MATH_COMPACT;
  Engine eng(math, split, ws, st);
  const int P = (int)ceil_div(C, NB);
  // Tensor path: the panel solve writes its result as bf16 planes too, and the rank-128 update
  // P P^T reads one plane set as both operands.
  const bool tensor = math == MQ_MATH_TENSOR;
  if (tensor) MQ_REQUIRE(split >= 1 && split <= 3, MQ_ERR_ARGUMENT, "factorisation: split must be 1, 2 or 3 (got %d)", split);
  {
    // ---- right-looking in two levels, last panel first.  Four panels form a super-panel of 512
    // columns.  Behind each panel only the columns of its own super-panel that are still to be
    // factored take their rank-128 update at once (a strip at most 384 wide); everything in
    // front of the super-panel is updated once per super-panel, with all 512 columns of it in one
    // contraction, so a tile of the trailing matrix is read and written once per 512 instead of
    // once per 128 eliminated columns.  Tensor path: the panel solve writes its result as bf16
    // planes too (k window of its panel inside a 512-wide plane buffer), and the updates read one
    // plane set as both operands.
    PlaneSet pset;
    if (tensor) {
      Workspace mine = eng.ws;
      pset.base = mine.take<uint16_t>(plane_set_bytes(C, SUPER_NB, split) / 2);
      MQ_REQUIRE(pset.base, MQ_ERR_WORKSPACE, "factorisation: workspace too small for the panel planes");
      pset.planes = split; pset.rows_pad = (int)pad_rows(C); pset.total_rows = pset.rows_pad; pset.K_pad = SUPER_NB;
    }
    for (int p = P - 1; p >= 0; --p) {
      const int p_lo = (p / SUPER_PANELS) * SUPER_PANELS;      // first (lowest) panel of this super-panel
      const int64_t k0 = (int64_t)p_lo * NB;                   // first column of the super-panel
      const int64_t k1 = (int64_t)p * NB;
      const int nb = (int)((C - k1) < NB ? (C - k1) : NB);
      const int kwin = (p - p_lo) * NB;                        // this panel's k window in the plane buffer
      float* dblk = H + k1 * ldh + k1;
      {
        ProfScope prof(PROF_CHOL_DIAG, (double)nb * nb * nb / 3.0, 0.0, st);
        MQ_CUDA(launch_chained(true, chol_diag_rev_kernel, dim3(1), dim3(DIAG_THREADS), kDiagSmem, st, dblk, ldh, nb, (int)k1, flags));
      }
      MQ_LAUNCH_CHECK();
      if (k1 == 0) break;
      // 32 rows per CTA (one group of four rows per warp); compact launches: 64 rows, half the CTAs
      // and half the copies of the diagonal block (462 against 454-459 layers/s on eight streams)
      const int grid = compact ? (int)ceil_div(k1, 64) : (int)(ceil_div(k1, 32) < 148 * 2 ? ceil_div(k1, 32) : 148 * 2);
      {
        ProfScope prof(PROF_TRSM, (double)k1 * nb * nb, 0.0, st);
        MQ_CUDA(launch_chained(true, trsm_rows_kernel<false>, dim3(grid, 1), dim3(256), kTrsmSmem, st, dblk, ldh, 0, H + k1, ldh, 0,
                               (int)k1, nb, 0, tensor ? pset.base + kwin : nullptr, tensor ? pset.total_rows * (int64_t)SUPER_NB : 0,
                               split, SUPER_NB));
      }
      MQ_LAUNCH_CHECK();
      if (!tensor) {
        GemmDesc g;
        g.A = H + k1; g.a_rs = ldh; g.a_cs = 1;
        g.B = H + k1; g.b_rs = 1; g.b_cs = ldh;
        g.C = H; g.ldc = ldh;
        g.M = (int)k1; g.N = (int)k1; g.K = nb;
        g.alpha = -1.0f; g.beta = 1.0f;
        g.upper_tiles_only = 1;
        MQ_TRY(eng.gemm(g));
        continue;
      }
      if (p > p_lo) {
        // near: H[0:k1, k0:k1] -= P P[k0:k1]^T, the rest of this super-panel
        GemmDesc g;
        g.C = H + k0; g.ldc = ldh;
        g.M = (int)k1; g.N = (int)(k1 - k0); g.K = nb;
        g.alpha = -1.0f; g.beta = 1.0f;
        g.compact = compact;
        PlaneSet a = pset, b = pset;
        a.k0 = kwin;
        b.k0 = kwin; b.row0 = k0;
        MQ_TRY(gemm_tensor_planes(g, a, b, st));
      } else if (k0 > 0) {
        // far: H[0:k0, 0:k0] -= P_S P_S^T over all columns of the super-panel, tiles on and above the diagonal
        const int p_hi = (p_lo + SUPER_PANELS - 1) < (P - 1) ? (p_lo + SUPER_PANELS - 1) : (P - 1);
        GemmDesc g;
        g.C = H; g.ldc = ldh;
        g.M = (int)k0; g.N = (int)k0; g.K = (p_hi - p_lo + 1) * NB;
        g.alpha = -1.0f; g.beta = 1.0f;
        g.upper_tiles_only = 1;
        g.k_round = NB;   // partial sums per panel meet in round-to-nearest adds, as in a one-level loop
        MQ_TRY(gemm_tensor_planes(g, pset, pset, st));
      }
    }
  }
  // ---- T -> unit-diagonal factor
  extract_diag_kernel<<<(unsigned)ceil_div(C, 256), 256, 0, st>>>(H, C, ldh, diag);
  MQ_LAUNCH_CHECK();
  {
    const int mode = unscaled ? 2 : (upper_only ? 1 : 0);
    const unsigned gx = unscaled ? 1u : (unsigned)(ceil_div(C, 256) < 8 ? ceil_div(C, 256) : 8);
    scale_columns_kernel<<<dim3(gx, (unsigned)C), unscaled ? 32 : 256, 0, st>>>(H, C, ldh, diag, mode);
    MQ_LAUNCH_CHECK();
  }
  identity_if_failed_kernel<<<148 * 4, 256, 0, st>>>(H, C, ldh, flags, diag);
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}

int hinv_upper(float* H, int64_t C, int64_t ldh, float* Uhat, int64_t ldu, float* diag_out, int math, int split,
               mq_layer_flags* flags, Workspace& ws, cudaStream_t st) {
  float* diag = ws.take<float>(C);
  float* scratch = ws.take<float>((size_t)C * C);
  MQ_REQUIRE(diag && scratch, MQ_ERR_WORKSPACE, "mq_hinv_upper: workspace too small");
  MQ_TRY(chol_unit_factor(H, C, ldh, diag, math, split, flags, ws, st, false, false));
  if (diag_out) MQ_CUDA(cudaMemcpyAsync(diag_out, diag, C * sizeof(float), cudaMemcpyDeviceToDevice, st));
  Engine eng(math, split, ws, st);
  const int P = (int)ceil_div(C, NB);
  // ---- inverse of the unit factor: invert the diagonal blocks, then merge pairs of blocks
  MQ_CUDA(cudaMemsetAsync(Uhat, 0, (size_t)C * ldu * sizeof(float), st));
  trsm_rows_kernel<true><<<dim3(4, P), 256, kTrsmSmem, st>>>(H, ldh, (int64_t)NB * (ldh + 1), Uhat, ldu,
                                                             (int64_t)NB * (ldu + 1), NB, NB, (int)C, nullptr, 0, 0, NB);
  MQ_LAUNCH_CHECK();
  for (int64_t s = NB; s < C; s *= 2) {
    const int batch = (int)ceil_div(C - s, 2 * s);
    GemmDesc g1;  // scratch block = B D^-1
    g1.A = H + s; g1.a_rs = ldh; g1.a_cs = 1; g1.a_bs = 2 * s * (ldh + 1);
    g1.B = Uhat + s * ldu + s; g1.b_rs = ldu; g1.b_cs = 1; g1.b_bs = 2 * s * (ldu + 1);
    g1.C = scratch + s; g1.ldc = C; g1.c_bs = 2 * s * (C + 1);
    g1.M = (int)s; g1.N = (int)s; g1.K = (int)s;
    g1.alpha = 1.0f; g1.beta = 0.0f;
    g1.b_upper = 1;
    g1.batch = batch; g1.n_total = (int)(C - s); g1.n_step = (int)(2 * s); g1.k_follows_n = 1;
    MQ_TRY(eng.gemm(g1));
    GemmDesc g2;  // off-diagonal block = -A^-1 (scratch block)
    g2.A = Uhat; g2.a_rs = ldu; g2.a_cs = 1; g2.a_bs = 2 * s * (ldu + 1);
    g2.B = scratch + s; g2.b_rs = C; g2.b_cs = 1; g2.b_bs = 2 * s * (C + 1);
    g2.C = Uhat + s; g2.ldc = ldu; g2.c_bs = 2 * s * (ldu + 1);
    g2.M = (int)s; g2.N = (int)s; g2.K = (int)s;
    g2.alpha = -1.0f; g2.beta = 0.0f;
    g2.a_upper = 1;
    g2.batch = batch; g2.n_total = (int)(C - s); g2.n_step = (int)(2 * s);
    MQ_TRY(eng.gemm(g2));
  }
  identity_if_failed_kernel<<<148 * 4, 256, 0, st>>>(Uhat, C, ldu, flags, diag);
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}

}  // namespace mq

extern "C" size_t mq_hinv_upper_workspace_bytes(int64_t C, int math, int split) {
  if (C <= 0) return 0;
  return mq::hinv_workspace_bytes(C, math, split);
}

extern "C" int mq_hinv_upper(float* H, int64_t C, int64_t ldh, float* Uhat, int64_t ldu, float* diag_out, int math, int split,
                             mq_layer_flags* flags, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace mq;
  MQ_REQUIRE(H && Uhat && flags, MQ_ERR_ARGUMENT, "mq_hinv_upper: null pointer");
  MQ_REQUIRE(C > 0 && ldh >= C && ldu >= C, MQ_ERR_ARGUMENT, "mq_hinv_upper: bad C=%lld ldh=%lld ldu=%lld", (long long)C,
             (long long)ldh, (long long)ldu);
  MQ_REQUIRE(C % 8 == 0, MQ_ERR_UNSUPPORTED, "mq_hinv_upper: C=%lld must be a multiple of 8", (long long)C);
  MQ_REQUIRE(ldh % 4 == 0 && ldu % 4 == 0 && aligned(H, 16) && aligned(Uhat, 16), MQ_ERR_ALIGNMENT,
             "mq_hinv_upper: H and Uhat must be 16-byte aligned with leading dimensions that are multiples of 4");
  MQ_REQUIRE(math == MQ_MATH_FP32 || math == MQ_MATH_TENSOR, MQ_ERR_ARGUMENT, "mq_hinv_upper: bad math %d", math);
  Workspace ws(workspace, workspace_bytes);
  return hinv_upper(H, C, ldh, Uhat, ldu, diag_out, math, split, flags, ws, static_cast<cudaStream_t>(stream));
}

extern "C" size_t mq_chol_unit_factor_workspace_bytes(int64_t C, int math, int split) {
  if (C <= 0) return 0;
  return mq::align_up((size_t)C * sizeof(float), 256) + mq::factor_workspace_bytes(C, math, split);
}

extern "C" int mq_chol_unit_factor(float* H, int64_t C, int64_t ldh, float* diag_out, int math, int split,
                                   mq_layer_flags* flags, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace mq;
  MQ_REQUIRE(H && flags, MQ_ERR_ARGUMENT, "mq_chol_unit_factor: null pointer");
  MQ_REQUIRE(C > 0 && ldh >= C, MQ_ERR_ARGUMENT, "mq_chol_unit_factor: bad C=%lld ldh=%lld", (long long)C, (long long)ldh);
  MQ_REQUIRE(C % 8 == 0, MQ_ERR_UNSUPPORTED, "mq_chol_unit_factor: C=%lld must be a multiple of 8", (long long)C);
  MQ_REQUIRE(ldh % 4 == 0 && aligned(H, 16), MQ_ERR_ALIGNMENT, "mq_chol_unit_factor: H must be 16-byte aligned, ldh %% 4 == 0");
  MQ_REQUIRE(math == MQ_MATH_FP32 || math == MQ_MATH_TENSOR, MQ_ERR_ARGUMENT, "mq_chol_unit_factor: bad math %d", math);
  Workspace ws(workspace, workspace_bytes);
  float* diag = ws.take<float>(C);
  MQ_REQUIRE(diag, MQ_ERR_WORKSPACE, "mq_chol_unit_factor: workspace too small");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MQ_TRY(chol_unit_factor(H, C, ldh, diag, math, split, flags, ws, st, false, false));
  if (diag_out) MQ_CUDA(cudaMemcpyAsync(diag_out, diag, C * sizeof(float), cudaMemcpyDeviceToDevice, st));
  return MQ_OK;
}
