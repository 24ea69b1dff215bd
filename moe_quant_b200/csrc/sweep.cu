// GPTQ column sweep.  Replaces the 2*C Triton launches and C/B cuBLAS calls of the
// reference's captured loop (src/gptq_loop.py:141-148) with, per 128-column tile,
// ONE sweep kernel plus ONE GEMM.
//
// Sweep kernel: a warp owns one weight row; lane l keeps columns 4l..4l+3 of the
// current tile in registers.  Column j is quantized by the lane that owns it
//   q = clamp(floor(x/s + z + 0.5), 0, maxq)   y = round_to_dtype((q - z) s)   e = y - x
// (src/gptq_loop.py:28-40, src/quant_utils.py:30-49), e is broadcast with one
// shuffle and every lane applies  w_k += Uhat[j,k] e  to its columns k > j with the
// row Uhat[j, tile] read from shared memory (src/gptq_loop.py:83-88).  Rows are
// independent, so there is no synchronisation after the tile of Uhat is staged.
//
// The errors of the tile (R x 128) go to a scratch matrix and the lazy update
//   W[:, later] += E Uhat[tile, later]             (src/gptq_loop.py:148)
// is a GEMM through the Engine.  Codes are written straight into the (R, C) uint8
// result, so the transposes of src/gptq.py:191-199 never happen.
#include "engine.cuh"
#include "profile.cuh"

namespace mq {

namespace {

constexpr int TILE = 128;
constexpr int SWEEP_THREADS = 512;  // 16 rows per CTA

template <int DT>
__global__ void __launch_bounds__(SWEEP_THREADS) sweep_tile_kernel(
    const float* __restrict__ W, int64_t ldw, int R, const float* __restrict__ U, int64_t ldu,
    const float* __restrict__ scale, const float* __restrict__ zero, int64_t group, int64_t s_rs, int64_t s_gs,
    float maxq, float zero_default, uint8_t* __restrict__ codes, int64_t C,
    typename StorageOf<DT>::type* __restrict__ deq, float* __restrict__ err, int i1, int nb,
    const float* __restrict__ Worig, int64_t ldwo, uint16_t* __restrict__ err_planes, int64_t plane_stride,
    int n_planes) {
  using T = typename StorageOf<DT>::type;
  extern __shared__ __align__(16) float ublk[];  // [TILE][TILE], strict upper triangle of the tile, 0 elsewhere
  // The factor is constant during the sweep: its tile is staged before this grid waits for the
  // rank-128 update that precedes it in the stream (only W depends on that update).
  for (int idx = threadIdx.x; idx < TILE * TILE / 4; idx += blockDim.x) {
    int j = idx >> 5, k4 = (idx & 31) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < nb && k4 < nb && k4 + 3 > j) {
      v = __ldg(reinterpret_cast<const float4*>(U + (int64_t)(i1 + j) * ldu + i1 + k4));
      if (k4 + 0 <= j) v.x = 0.f;
      if (k4 + 1 <= j) v.y = 0.f;
      if (k4 + 2 <= j) v.z = 0.f;
    }
    *reinterpret_cast<float4*>(&ublk[j * TILE + k4]) = v;
  }
  chain_wait();
  chain_release();
  __syncthreads();

  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * (SWEEP_THREADS / 32) + (threadIdx.x >> 5);
  if (r >= R) return;
  const int c0 = i1 + lane * 4;
  const bool have = lane * 4 < nb;  // nb is a multiple of 4

  float w[4] = {0.f, 0.f, 0.f, 0.f}, sc[4] = {1.f, 1.f, 1.f, 1.f}, zr[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) zr[t] = zero_default;
  if (have) {
    float4 v = *reinterpret_cast<const float4*>(W + (int64_t)r * ldw + c0);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    const int grp = (int)group;
    if ((grp & 3) == 0) {
      // the four columns of a lane share a group: one index, one 32-bit division
      const int64_t off = (int64_t)r * s_rs + (int64_t)(c0 / grp) * s_gs;
      const float s0 = __ldg(scale + off);
      const float z0 = zero ? __ldg(zero + off) : zero_default;
#pragma unroll
      for (int t = 0; t < 4; ++t) { sc[t] = s0; zr[t] = z0; }
    } else {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int64_t off = (int64_t)r * s_rs + (int64_t)((c0 + t) / grp) * s_gs;
        sc[t] = __ldg(scale + off);
        if (zero) zr[t] = __ldg(zero + off);
      }
    }
  }
  float qv[4] = {0.f, 0.f, 0.f, 0.f}, yv[4] = {0.f, 0.f, 0.f, 0.f}, ev[4] = {0.f, 0.f, 0.f, 0.f};
  // Inverse-free form (Worig != nullptr): U is the unit factor Utilde = Uhat^-1 and what is
  // propagated is minus the total change of the column, -(y - w_original), instead of the
  // error against the running value; x_j = w_j - sum_{i<j} (y_i - w_i) Utilde[i,j] is the same
  // number as the reference's running weight (E Uhat = Y - W  <=>  E = (Y - W) Utilde).
  const bool inverse_free = Worig != nullptr;
  float wo[4] = {0.f, 0.f, 0.f, 0.f};
  if (inverse_free && have) {
    float4 v = *reinterpret_cast<const float4*>(Worig + (int64_t)r * ldwo + c0);
    wo[0] = v.x; wo[1] = v.y; wo[2] = v.z; wo[3] = v.w;
  }

  // x / s through the reciprocal and one correction step (the final stage of a correctly rounded
  // division): a few FMAs on the serial chain instead of the full division sequence.
  float rs[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) rs[t] = 1.0f / sc[t];

  const int n_quads = nb >> 2;
  for (int jq = 0; jq < n_quads; ++jq) {
    // The four columns of quad jq belong to lane jq and depend on each other only through the
    // 4 x 4 diagonal block of U, so that lane can run them back to back without a shuffle.  Every
    // lane runs the same four steps on a copy of its own values against that block (uniform
    // code, no divergence); only lane jq's results are real.  Its four errors are then broadcast
    // and applied to the true running weights of all lanes, in the same order, with the same
    // FMAs the one-column-at-a-time recurrence would use.
    float wl[4] = {w[0], w[1], w[2], w[3]};
    float e4[4];
    const float* ud = &ublk[(jq * 4) * TILE + jq * 4];  // diagonal block, same address for all lanes
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float x = wl[t];
      float d = x * rs[t];
      d = fmaf(fmaf(-sc[t], d, x), rs[t], d);
      const float q = fminf(fmaxf(floorf((d + zr[t]) + 0.5f), 0.0f), maxq);
      const float y = round_through<DT>((q - zr[t]) * sc[t]);
      const float e = inverse_free ? (wo[t] - y) : (y - x);
      e4[t] = e;
      if (lane == jq) { qv[t] = q; yv[t] = y; ev[t] = e; }
#pragma unroll
      for (int t2 = t + 1; t2 < 4; ++t2) wl[t2] = fmaf(ud[t * TILE + t2], e, wl[t2]);
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float eb = __shfl_sync(0xffffffffu, e4[t], jq);
      const float4 u = *reinterpret_cast<const float4*>(&ublk[(jq * 4 + t) * TILE + lane * 4]);
      w[0] = fmaf(u.x, eb, w[0]);
      w[1] = fmaf(u.y, eb, w[1]);
      w[2] = fmaf(u.z, eb, w[2]);
      w[3] = fmaf(u.w, eb, w[3]);
    }
  }
  if (have) {
    uchar4 qc = make_uchar4((unsigned char)qv[0], (unsigned char)qv[1], (unsigned char)qv[2], (unsigned char)qv[3]);
    *reinterpret_cast<uchar4*>(codes + (int64_t)r * C + c0) = qc;
    if (deq) {
#pragma unroll
      for (int t = 0; t < 4; ++t) deq[(int64_t)r * C + c0 + t] = from_float<T>(yv[t]);
    }
  }
  // columns past nb of a narrow last tile hold zeros so the GEMM may read all 128
  if (err_planes) {
    // the tensor-core update reads the errors as bf16 planes: write them in that form directly
    uint16_t h[4], m[4], l[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) split_bf16x3(ev[t], h[t], m[t], l[t]);
    uint16_t* dst = err_planes + (int64_t)r * TILE + lane * 4;
    *reinterpret_cast<uint2*>(dst) = make_uint2((uint32_t)h[0] | ((uint32_t)h[1] << 16), (uint32_t)h[2] | ((uint32_t)h[3] << 16));
    if (n_planes > 1)
      *reinterpret_cast<uint2*>(dst + plane_stride) =
          make_uint2((uint32_t)m[0] | ((uint32_t)m[1] << 16), (uint32_t)m[2] | ((uint32_t)m[3] << 16));
    if (n_planes > 2)
      *reinterpret_cast<uint2*>(dst + 2 * plane_stride) =
          make_uint2((uint32_t)l[0] | ((uint32_t)l[1] << 16), (uint32_t)l[2] | ((uint32_t)l[3] << 16));
  } else {
    *reinterpret_cast<float4*>(err + (int64_t)r * TILE + lane * 4) = make_float4(ev[0], ev[1], ev[2], ev[3]);
  }
}

int configure_once() {
  static bool done[64] = {};
  int dev = 0;
  MQ_CUDA(cudaGetDevice(&dev));
  if (!done[dev & 63]) {
    const int bytes = TILE * TILE * (int)sizeof(float);
    MQ_CUDA(cudaFuncSetAttribute(sweep_tile_kernel<MQ_F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    MQ_CUDA(cudaFuncSetAttribute(sweep_tile_kernel<MQ_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    MQ_CUDA(cudaFuncSetAttribute(sweep_tile_kernel<MQ_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done[dev & 63] = true;
  }
  return MQ_OK;
}

}  // namespace

size_t sweep_workspace_bytes(int64_t R, int64_t C, int math, int split) {
  size_t bytes = align_up((size_t)R * TILE * sizeof(float), 256);
  if (math == MQ_MATH_TENSOR) bytes += plane_set_bytes(R, TILE, split) + plane_set_bytes(C, C, split);
  return bytes;
}

int gptq_sweep(float* W, int64_t R, int64_t C, int64_t ldw, const float* Uhat, int64_t ldu, const float* scale,
               const float* zero, int64_t group, int64_t s_rs, int64_t s_gs, int bits, int out_dtype, uint8_t* codes,
               void* deq, const float* Worig, int64_t ldwo, int math, int split, Workspace& ws, cudaStream_t st,
               const float* col_div) {
  // col_div (tensor math only): above its diagonal 128-blocks Uhat holds the factor before its
  // columns were divided by col_div; the plane split divides where it reads it.  The diagonal
  // blocks, which the tiles read, are already scaled.
  MQ_TRY(configure_once());
  float* err = ws.take<float>((size_t)R * TILE);
  MQ_REQUIRE(err, MQ_ERR_WORKSPACE, "mq_gptq_sweep: workspace too small");
  Engine eng(math, split, ws, st);
  // Tensor path: the factor is cut into transposed planes once (row n, k -> U[k][n]); the lazy
  // update of tile i1 then reads the window k in [i1, i1+128), rows n >= i2 of those planes,
  // and the sweep kernel writes its errors as planes itself.  No per-tile conversion passes.
  PlaneSet err_set, u_set;
  const bool tensor = math == MQ_MATH_TENSOR;
  if (tensor) {
    MQ_REQUIRE(split >= 1 && split <= 3, MQ_ERR_ARGUMENT, "mq_gptq_sweep: split must be 1, 2 or 3 (got %d)", split);
    uint16_t* ep = ws.take<uint16_t>(plane_set_bytes(R, TILE, split) / 2);
    uint16_t* up = ws.take<uint16_t>(plane_set_bytes(C, C, split) / 2);
    MQ_REQUIRE(ep && up, MQ_ERR_WORKSPACE, "mq_gptq_sweep: workspace too small for the operand planes");
    err_set.base = ep; err_set.planes = split; err_set.rows_pad = (int)pad_rows(R); err_set.total_rows = err_set.rows_pad;
    err_set.K_pad = TILE;
    // the lazy updates read Uhat[i1:i2, i2:]: only blocks strictly above the diagonal
    MQ_TRY(make_planes_f32(Uhat, 1, ldu, (int)C, (int)C, split, up, &u_set, st, true, col_div));
  }
  uint16_t* const ep_arg = tensor ? err_set.base : nullptr;
  const int64_t ep_stride = tensor ? err_set.total_rows * TILE : 0;
  const float maxq = (float)((1 << bits) - 1);
  const float zero_default = 0.5f * (float)(1 << bits);
  const int grid = (int)ceil_div(R, SWEEP_THREADS / 32);
  const size_t smem = TILE * TILE * sizeof(float);
  for (int64_t i1 = 0; i1 < C; i1 += TILE) {
    const int nb = (int)((C - i1) < TILE ? (C - i1) : TILE);
    // bytes the tile must move: W in, codes out, errors out, the triangle of Uhat once
    {
    // The kernel stages its tile of the factor before it waits for its predecessor: only a launch
    // that follows this loop's own update (which writes W, never the factor) may be chained.
    const bool chained = i1 > 0;
    ProfScope prof(PROF_SWEEP_TILE, (double)R * nb * (4.0 + 1.0 + 4.0) + 2.0 * nb * nb, (double)R * nb * (nb - 1), st);
    switch (out_dtype) {
      case MQ_F32:
        MQ_CUDA(launch_chained(chained, sweep_tile_kernel<MQ_F32>, dim3(grid), dim3(SWEEP_THREADS), smem, st, W, ldw, (int)R, Uhat, ldu, scale, zero, group, s_rs, s_gs,
                                                                  maxq, zero_default, codes, C, static_cast<float*>(deq), err,
                                                                  (int)i1, nb, Worig, ldwo, ep_arg, ep_stride, split));
        break;
      case MQ_BF16:
        MQ_CUDA(launch_chained(chained, sweep_tile_kernel<MQ_BF16>, dim3(grid), dim3(SWEEP_THREADS), smem, st, W, ldw, (int)R, Uhat, ldu, scale, zero, group, s_rs, s_gs,
                                                                   maxq, zero_default, codes, C,
                                                                   static_cast<__nv_bfloat16*>(deq), err, (int)i1, nb, Worig, ldwo, ep_arg, ep_stride, split));
        break;
      default:
        MQ_CUDA(launch_chained(chained, sweep_tile_kernel<MQ_F16>, dim3(grid), dim3(SWEEP_THREADS), smem, st, W, ldw, (int)R, Uhat, ldu, scale, zero, group, s_rs, s_gs,
                                                                  maxq, zero_default, codes, C, static_cast<__half*>(deq), err,
                                                                  (int)i1, nb, Worig, ldwo, ep_arg, ep_stride, split));
    }
    }
    MQ_LAUNCH_CHECK();
    const int64_t i2 = i1 + nb;
    if (i2 < C) {
      GemmDesc g;
      g.A = err; g.a_rs = TILE; g.a_cs = 1;
      g.B = Uhat + i1 * ldu + i2; g.b_rs = ldu; g.b_cs = 1;
      g.C = W + i2; g.ldc = ldw;
      g.M = (int)R; g.N = (int)(C - i2); g.K = nb;
      g.alpha = 1.0f; g.beta = 1.0f;
      if (tensor) {
        PlaneSet b = u_set;
        b.row0 = i2;
        b.k0 = (int)i1;
        MQ_TRY(gemm_tensor_planes(g, err_set, b, st));
      } else {
        MQ_TRY(eng.gemm(g));
      }
    }
  }
  return MQ_OK;
}

}  // namespace mq

extern "C" size_t mq_gptq_sweep_workspace_bytes(int64_t R, int64_t C, int math, int split) {
  if (R <= 0 || C <= 0) return 0;
  return mq::sweep_workspace_bytes(R, C, math, split);
}

extern "C" int mq_gptq_sweep(float* W, int64_t R, int64_t C, int64_t ldw, const float* Uhat, int64_t ldu,
                             const float* scale, const float* zero, int64_t group, int64_t row_stride,
                             int64_t group_stride, int bits, int out_dtype, uint8_t* codes, void* dequantized,
                             const float* W_original, int64_t ldwo, int math, int split, void* workspace,
                             size_t workspace_bytes, void* stream) {
  using namespace mq;
  MQ_REQUIRE(W && Uhat && scale && codes, MQ_ERR_ARGUMENT, "mq_gptq_sweep: null pointer");
  MQ_REQUIRE(R > 0 && C > 0 && ldw >= C && ldu >= C, MQ_ERR_ARGUMENT, "mq_gptq_sweep: bad shape R=%lld C=%lld ldw=%lld ldu=%lld",
             (long long)R, (long long)C, (long long)ldw, (long long)ldu);
  MQ_REQUIRE(group > 0 && C % group == 0, MQ_ERR_ARGUMENT, "mq_gptq_sweep: group %lld does not divide C=%lld", (long long)group,
             (long long)C);
  MQ_REQUIRE(bits >= 2 && bits <= 8, MQ_ERR_ARGUMENT, "mq_gptq_sweep: bits=%d", bits);
  MQ_REQUIRE(valid_dtype(out_dtype), MQ_ERR_ARGUMENT, "mq_gptq_sweep: bad dtype %d", out_dtype);
  MQ_REQUIRE(C % 8 == 0, MQ_ERR_UNSUPPORTED, "mq_gptq_sweep: C=%lld must be a multiple of 8", (long long)C);
  MQ_REQUIRE(ldw % 4 == 0 && ldu % 4 == 0 && aligned(W, 16) && aligned(Uhat, 16) && aligned(codes, 4), MQ_ERR_ALIGNMENT,
             "mq_gptq_sweep: W/Uhat need 16-byte alignment and leading dimensions that are multiples of 4");
  MQ_REQUIRE(math == MQ_MATH_FP32 || math == MQ_MATH_TENSOR, MQ_ERR_ARGUMENT, "mq_gptq_sweep: bad math %d", math);
  Workspace ws(workspace, workspace_bytes);
  if (W_original) {
    MQ_REQUIRE(ldwo >= C && ldwo % 4 == 0 && aligned(W_original, 16) && W_original != W, MQ_ERR_ALIGNMENT,
               "mq_gptq_sweep: W_original must be a separate 16-byte aligned matrix with ldwo %% 4 == 0");
  }
  return gptq_sweep(W, R, C, ldw, Uhat, ldu, scale, zero, group, row_stride, group_stride, bits, out_dtype, codes,
                    dequantized, W_original, ldwo, math, split, ws, static_cast<cudaStream_t>(stream), nullptr);
}
