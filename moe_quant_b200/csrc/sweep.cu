// GPTQ column sweep.  Replaces the 2*C Triton launches and C/B cuBLAS calls of the
// reference's captured loop (src/gptq_loop.py:141-148) with, per 128-column tile,
// ONE sweep kernel plus ONE GEMM.
//
// Sweep kernel: sixteen lanes share one weight row, lane l keeps columns 8l..8l+7 of the
// current tile in registers (two rows per warp).  Column j is quantized as
//   q = clamp(floor(x/s + z + 0.5), 0, maxq)   y = round_to_dtype((q - z) s)   e = y - x
// (src/gptq_loop.py:28-40, src/quant_utils.py:30-49) and its error is applied to the columns
// behind it, w_k += Uhat[j,k] e (src/gptq_loop.py:83-88), with one fma per (j, k) in
// increasing j: the reference's order.  The eight columns of a lane are a chain that needs
// no communication (the lane applies each error to its own later columns at once), so the
// tile is sixteen such chains back to back; after a chain its eight errors are broadcast with
// shuffles and the other lanes of the row apply them to their columns.  Rows are independent:
// no block-wide synchronisation after the tile of Uhat is staged in shared memory.
// (sweep_rows.cuh holds the same tile with one row per thread, for callers that run several
// layers at once.)
//
// The errors of the tile (R x 128) go to a scratch matrix, as bf16 planes on the tensor path,
// and the lazy update
//   W[:, later] += E Uhat[tile, later]             (src/gptq_loop.py:148)
// is a GEMM: on the tensor path in two levels (the rest of the tile's 512-column super-block at
// once, everything behind the super-block once per super-block with all 512 errors of a row
// in the contraction), on the fp32 path one update of everything behind the tile.  Codes are
// written straight into the (R, C) uint8 result, so the transposes of src/gptq.py:191-199
// never happen.
#include "engine.cuh"
#include "profile.cuh"
#include "sweep.cuh"
#include "sweep_rows.cuh"

namespace mq {

namespace {

constexpr int TILE = SWEEP_TILE;
constexpr int TILE_THREADS = 128;                        // threads per CTA of the lane-per-chunk kernel
// LANES lanes share one weight row and keep TILE / LANES consecutive columns each.  Sixteen lanes
// (8 columns, 8 rows per CTA) give the shorter serial stream per warp: 4.83 against 5.03 ms per
// 2048 x 7168 layer on one stream (with 256 threads per CTA 4.95 ms); a layer with more rows than
// the grid holds at that shape walks its row groups in turns, and eight lanes (16 columns, 16 rows
// per CTA) are faster again (7168 x 2048: 623 against 586 layers/s).  4 columns per lane would
// need shuffles to form the 8-column vectors in which codes, packed words and error planes leave.
// The tile of the factor in shared memory: row j holds LANES chunks, 4 floats of padding after
// each, so that the lanes of a quarter-warp read their 16-byte pieces from disjoint banks.
template <int LANES>
struct LaneShape {
  static constexpr int ROW_LANES = LANES;
  static constexpr int LANE_COLS = TILE / LANES;
  static constexpr int U_LANE_LD = LANE_COLS + 4;
  static constexpr int U_ROW_LD = LANES * U_LANE_LD;       // 160 floats for 8 lanes, 192 for 16
  static constexpr size_t smem = (size_t)TILE * U_ROW_LD * sizeof(float);
};
constexpr int MAX_SWEEP_CTAS = 2 * 148;
// Four tiles form a super-block of 512 columns.  Behind each tile only the rest of its own
// super-block takes the rank-128 update at once; the columns behind the super-block are updated
// once per super-block with all 512 errors of a row in one contraction, so a tile of W is read
// and written once per 512 instead of once per 128 swept columns.
constexpr int SUPER = 4 * TILE;

// One 128 x 128 tile of the factor (top-left element at `src`) -> shared memory in the chunked
// row layout, strict upper triangle only.  stage: issue the copies (asynchronous 16-byte copies,
// all in flight at once; a copy with source size 0 writes zeros: everything below the diagonal
// and past nb); trim: wait for them and zero the entries on and below the diagonal inside each
// row's diagonal quad.  Every thread of the CTA must call both.
template <int LANES>
__device__ __forceinline__ void stage_factor_tile(float* ublk, const float* __restrict__ src, int64_t ldu, int nb) {
  constexpr int LANE_COLS = LaneShape<LANES>::LANE_COLS, U_LANE_LD = LaneShape<LANES>::U_LANE_LD, U_ROW_LD = LaneShape<LANES>::U_ROW_LD;
  for (int idx = threadIdx.x; idx < TILE * TILE / 4; idx += blockDim.x) {
    const int j = idx >> 5, k4 = (idx & 31) * 4;
    const bool keep = j < nb && k4 < nb && k4 + 3 > j;
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&ublk[j * U_ROW_LD + (k4 / LANE_COLS) * U_LANE_LD + (k4 % LANE_COLS)]);
    const float* g = keep ? src + (int64_t)j * ldu + k4 : src;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(g), "r"(keep ? 16 : 0) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

template <int LANES>
__device__ __forceinline__ void trim_factor_tile(float* ublk, int nb) {
  constexpr int LANE_COLS = LaneShape<LANES>::LANE_COLS, U_LANE_LD = LaneShape<LANES>::U_LANE_LD, U_ROW_LD = LaneShape<LANES>::U_ROW_LD;
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  for (int j = threadIdx.x; j < nb; j += blockDim.x) {
    const int k4 = j & ~3;
    float* q = &ublk[j * U_ROW_LD + (k4 / LANE_COLS) * U_LANE_LD + (k4 % LANE_COLS)];
    for (int k = 0; k <= (j & 3); ++k) q[k] = 0.0f;
  }
  __syncthreads();
}

// UNIFORM: the columns of a lane lie in one quantization group (group % LANE_COLS == 0).
template <int DT, bool UNIFORM, int LANES>
__global__ void __launch_bounds__(TILE_THREADS) sweep_tile_kernel(const SweepArgs a) {
  constexpr int ROW_LANES = LANES, LANE_COLS = LaneShape<LANES>::LANE_COLS;
  constexpr int U_LANE_LD = LaneShape<LANES>::U_LANE_LD, U_ROW_LD = LaneShape<LANES>::U_ROW_LD;
  constexpr int ROWS_PER_CTA = TILE_THREADS / ROW_LANES;
  using T = typename StorageOf<DT>::type;
  extern __shared__ __align__(16) float ublk[];  // [TILE][U_ROW_LD], strict upper triangle of the tile, 0 elsewhere
  const int nb = a.nb, i1 = a.i1;
  // The factor is constant during the sweep: its tile is staged before this grid waits for the
  // rank-128 update that precedes it in the stream (only W depends on that update).
  stage_factor_tile<LANES>(ublk, a.U + (int64_t)i1 * a.ldu + i1, a.ldu, nb);
  chain_wait();
  chain_release();
  trim_factor_tile<LANES>(ublk, nb);

  const int sub = threadIdx.x & (ROW_LANES - 1);   // this lane's chunk of the row
  const int c_local = sub * LANE_COLS;
  const int c0 = i1 + c_local;
  const float maxq = a.maxq;
  // Inverse-free form (Worig != nullptr): U is the unit factor Utilde = Uhat^-1 and what is
  // propagated is minus the total change of the column, -(y - w_original), instead of the
  // error against the running value; x_j = w_j - sum_{i<j} (y_i - w_i) Utilde[i,j] is the same
  // number as the reference's running weight (E Uhat = Y - W  <=>  E = (Y - W) Utilde).
  const bool inverse_free = a.Worig != nullptr;
  const int n_owner = (nb + LANE_COLS - 1) / LANE_COLS;
  const int row_groups = (a.R + ROWS_PER_CTA - 1) / ROWS_PER_CTA;

  // the CTA walks row groups together (the shuffles below are warp-wide); rows past R carry zeros
  for (int rg = blockIdx.x; rg < row_groups; rg += gridDim.x) {
    const int r = rg * ROWS_PER_CTA + (threadIdx.x / ROW_LANES);
    const bool valid = r < a.R;
    float w[LANE_COLS], wo[LANE_COLS];
#pragma unroll
    for (int qd = 0; qd < LANE_COLS / 4; ++qd) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f), vo = v;
      if (valid && c_local + 4 * qd < nb) {
        v = *reinterpret_cast<const float4*>(a.W + (int64_t)r * a.ldw + c0 + 4 * qd);
        if (inverse_free) vo = *reinterpret_cast<const float4*>(a.Worig + (int64_t)r * a.ldwo + c0 + 4 * qd);
      }
      w[4 * qd] = v.x; w[4 * qd + 1] = v.y; w[4 * qd + 2] = v.z; w[4 * qd + 3] = v.w;
      wo[4 * qd] = vo.x; wo[4 * qd + 1] = vo.y; wo[4 * qd + 2] = vo.z; wo[4 * qd + 3] = vo.w;
    }
    // grid of the lane's columns; x / s goes through the reciprocal and one correction step (the
    // final stage of a correctly rounded division): a few FMAs on the serial chain instead of
    // the full division sequence
    constexpr int NS = UNIFORM ? 1 : LANE_COLS;
    float sc[NS], zr[NS], rs[NS];
#pragma unroll
    for (int t = 0; t < NS; ++t) {
      sc[t] = 1.0f;
      zr[t] = a.zero_default;
      if (valid && c_local + t < nb) {
        const int64_t off = (int64_t)r * a.s_rs + (int64_t)((c0 + t) / a.group) * a.s_gs;
        sc[t] = __ldg(a.scale + off);
        if (a.zero) zr[t] = __ldg(a.zero + off);
      }
      rs[t] = 1.0f / sc[t];
    }
    // what this lane produces when its turn comes: the errors of its columns and their
    // codes, two to a float (q0 + 256 q1 is exact for codes below 256)
    float e[LANE_COLS], qacc[LANE_COLS / 2];
#pragma unroll
    for (int t = 0; t < LANE_COLS; ++t) e[t] = 0.0f;
#pragma unroll
    for (int h = 0; h < LANE_COLS / 2; ++h) qacc[h] = 0.0f;

#pragma unroll 1
    for (int lo = 0; lo < n_owner; ++lo) {
      if (sub == lo) {
        // Chain of this lane's columns against its diagonal LANE_COLS x LANE_COLS block of the factor
        // (the lanes of the warp that own chunk `lo` of their rows run it; the others wait).
        // A step applies the error to the whole quad rows behind it: entries on and below the
        // diagonal are zero in the staged tile and the columns they touch are finished.
        const float* ud = &ublk[(lo * LANE_COLS) * U_ROW_LD + lo * U_LANE_LD];
#pragma unroll
        for (int t = 0; t < LANE_COLS; ++t) {
          const float s_t = sc[UNIFORM ? 0 : t], z_t = zr[UNIFORM ? 0 : t], r_t = rs[UNIFORM ? 0 : t];
          const float x = w[t];
          float d = x * r_t;
          d = fmaf(fmaf(-s_t, d, x), r_t, d);
          const float q = fminf(fmaxf(floorf((d + z_t) + 0.5f), 0.0f), maxq);
          const float y = round_through<DT>((q - z_t) * s_t);
          const float et = inverse_free ? (wo[t] - y) : (y - x);
          e[t] = et;
          qacc[t >> 1] = (t & 1) ? fmaf(q, 256.0f, qacc[t >> 1]) : q;
          const float2 e2 = make_float2(et, et);
#pragma unroll
          for (int qd = (t + 1) >> 2; qd < LANE_COLS / 4; ++qd) {
            const float4 u = *reinterpret_cast<const float4*>(&ud[t * U_ROW_LD + 4 * qd]);
            const float2 p01 = __ffma2_rn(make_float2(u.x, u.y), e2, make_float2(w[4 * qd], w[4 * qd + 1]));
            const float2 p23 = __ffma2_rn(make_float2(u.z, u.w), e2, make_float2(w[4 * qd + 2], w[4 * qd + 3]));
            w[4 * qd] = p01.x; w[4 * qd + 1] = p01.y; w[4 * qd + 2] = p23.x; w[4 * qd + 3] = p23.y;
          }
        }
      }
      __syncwarp();
      // The errors of lane lo reach the other lanes of the row, which apply them to their
      // own columns in the same order, with the same FMAs, as a one-column-at-a-time recurrence.
      // (For the lanes in front of lo the staged factor holds zeros; lane lo's own values are
      // not needed any more.)
#pragma unroll
      for (int t = 0; t < LANE_COLS; ++t) {
        const float eb = __shfl_sync(0xffffffffu, e[t], lo, ROW_LANES);
        const float4* up = reinterpret_cast<const float4*>(&ublk[(lo * LANE_COLS + t) * U_ROW_LD + sub * U_LANE_LD]);
        const float2 eb2 = make_float2(eb, eb);
#pragma unroll
        for (int qd = 0; qd < LANE_COLS / 4; ++qd) {
          // packed fp32 FMA: two columns per instruction, each half an ordinary fma.rn
          const float4 u = up[qd];
          const float2 p01 = __ffma2_rn(make_float2(u.x, u.y), eb2, make_float2(w[4 * qd], w[4 * qd + 1]));
          const float2 p23 = __ffma2_rn(make_float2(u.z, u.w), eb2, make_float2(w[4 * qd + 2], w[4 * qd + 3]));
          w[4 * qd] = p01.x; w[4 * qd + 1] = p01.y; w[4 * qd + 2] = p23.x; w[4 * qd + 3] = p23.y;
        }
      }
    }

    // ---- every lane writes what its columns produced
    if (valid) {
#pragma unroll
      for (int qd = 0; qd < LANE_COLS / 4; ++qd) {
        if (c_local + 4 * qd >= nb) continue;
        const uint32_t q4 = (uint32_t)qacc[2 * qd] | ((uint32_t)qacc[2 * qd + 1] << 16);   // four codes, one per byte, first column lowest
        *reinterpret_cast<uint32_t*>(a.codes + (int64_t)r * a.C + c0 + 4 * qd) = q4;
        if (a.deq) {
          T* dq = static_cast<T*>(a.deq) + (int64_t)r * a.C + c0 + 4 * qd;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float qf = (float)((q4 >> (8 * t)) & 0xFFu);
            dq[t] = from_float<T>((qf - zr[UNIFORM ? 0 : 4 * qd + t]) * sc[UNIFORM ? 0 : 4 * qd + t]);
          }
        }
      }
      if (a.packed) {
        // the compressed-tensors word of columns 8k..8k+7 (column 8k+i at bits 4i..4i+3), written
        // here so that no separate packing pass has to read the codes back
#pragma unroll
        for (int h = 0; h < LANE_COLS / 8; ++h) {
          if (c_local + 8 * h >= nb) continue;
          const uint32_t lo4 = (uint32_t)qacc[4 * h] | ((uint32_t)qacc[4 * h + 1] << 16);
          const uint32_t hi4 = (uint32_t)qacc[4 * h + 2] | ((uint32_t)qacc[4 * h + 3] << 16);
          a.packed[(int64_t)r * (a.C >> 3) + ((c0 + 8 * h) >> 3)] = (int32_t)pack_nibbles(lo4, hi4);
        }
      }
      // columns past nb of a narrow last tile hold zeros so that the GEMM may read all 128
      if (a.err_planes) {
        // the tensor-core update reads the errors as bf16 planes: write them in that form directly
        uint32_t hp[LANE_COLS / 2], mp[LANE_COLS / 2], lp[LANE_COLS / 2];
#pragma unroll
        for (int t = 0; t < LANE_COLS; t += 2) {
          uint16_t h0, m0, l0, h1, m1, l1;
          split_bf16x3(e[t], h0, m0, l0);
          split_bf16x3(e[t + 1], h1, m1, l1);
          hp[t >> 1] = (uint32_t)h0 | ((uint32_t)h1 << 16);
          mp[t >> 1] = (uint32_t)m0 | ((uint32_t)m1 << 16);
          lp[t >> 1] = (uint32_t)l0 | ((uint32_t)l1 << 16);
        }
        uint16_t* dst = a.err_planes + (int64_t)r * a.err_ld + c_local;
#pragma unroll
        for (int v = 0; v < LANE_COLS / 8; ++v) {
          reinterpret_cast<uint4*>(dst)[v] = make_uint4(hp[4 * v], hp[4 * v + 1], hp[4 * v + 2], hp[4 * v + 3]);
          if (a.n_planes > 1)
            reinterpret_cast<uint4*>(dst + a.plane_stride)[v] = make_uint4(mp[4 * v], mp[4 * v + 1], mp[4 * v + 2], mp[4 * v + 3]);
          if (a.n_planes > 2)
            reinterpret_cast<uint4*>(dst + 2 * a.plane_stride)[v] = make_uint4(lp[4 * v], lp[4 * v + 1], lp[4 * v + 2], lp[4 * v + 3]);
        }
      } else {
        float4* dst = reinterpret_cast<float4*>(a.err + (int64_t)r * a.err_ld + c_local);
#pragma unroll
        for (int qd = 0; qd < LANE_COLS / 4; ++qd) dst[qd] = make_float4(e[4 * qd], e[4 * qd + 1], e[4 * qd + 2], e[4 * qd + 3]);
      }
    }
  }
}

template <int DT>
int launch_sweep_tile(bool chained, bool uniform, int lanes, int grid, cudaStream_t st, const SweepArgs& args) {
  if (lanes == 16) {
    if (uniform) MQ_CUDA(launch_chained(chained, sweep_tile_kernel<DT, true, 16>, dim3(grid), dim3(TILE_THREADS), LaneShape<16>::smem, st, args));
    else MQ_CUDA(launch_chained(chained, sweep_tile_kernel<DT, false, 16>, dim3(grid), dim3(TILE_THREADS), LaneShape<16>::smem, st, args));
  } else {
    if (uniform) MQ_CUDA(launch_chained(chained, sweep_tile_kernel<DT, true, 8>, dim3(grid), dim3(TILE_THREADS), LaneShape<8>::smem, st, args));
    else MQ_CUDA(launch_chained(chained, sweep_tile_kernel<DT, false, 8>, dim3(grid), dim3(TILE_THREADS), LaneShape<8>::smem, st, args));
  }
  return MQ_OK;
}

template <int DT>
int configure_dtype() {
  MQ_CUDA(cudaFuncSetAttribute(sweep_tile_kernel<DT, true, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LaneShape<8>::smem));
  MQ_CUDA(cudaFuncSetAttribute(sweep_tile_kernel<DT, false, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LaneShape<8>::smem));
  MQ_CUDA(cudaFuncSetAttribute(sweep_tile_kernel<DT, true, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LaneShape<16>::smem));
  MQ_CUDA(cudaFuncSetAttribute(sweep_tile_kernel<DT, false, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)LaneShape<16>::smem));
  return MQ_OK;
}

int configure_once() {
  static bool done[64] = {};
  int dev = 0;
  MQ_CUDA(cudaGetDevice(&dev));
  if (!done[dev & 63]) {
    MQ_TRY(configure_dtype<MQ_F32>());
    MQ_TRY(configure_dtype<MQ_BF16>());
    MQ_TRY(configure_dtype<MQ_F16>());
    done[dev & 63] = true;
  }
  return MQ_OK;
}

}  // namespace

size_t sweep_workspace_bytes(int64_t R, int64_t C, int math, int split) {
  math &= ~MQ_MATH_COMPACT;
  if (math == MQ_MATH_TENSOR) return plane_set_bytes(R, SUPER, split) + plane_set_bytes(C, C, split);
  return align_up((size_t)R * TILE * sizeof(float), 256);
}

int gptq_sweep(float* W, int64_t R, int64_t C, int64_t ldw, const float* Uhat, int64_t ldu, const float* scale,
               const float* zero, int64_t group, int64_t s_rs, int64_t s_gs, int bits, int out_dtype, uint8_t* codes,
               void* deq, const float* Worig, int64_t ldwo, int math, int split, Workspace& ws, cudaStream_t st,
               const float* col_div, int32_t* packed) {
  // col_div (tensor math only): above its diagonal 128-blocks Uhat holds the factor before its
  // columns were divided by col_div; the plane split divides where it reads it.  The diagonal
  // blocks, which the tiles read, are already scaled.
  MQ_TRY(configure_once());
  const bool compact = (math & MQ_MATH_COMPACT) != 0;
  math &= ~MQ_MATH_COMPACT;
  const bool tensor = math == MQ_MATH_TENSOR;
  float* err = tensor ? nullptr : ws.take<float>((size_t)R * TILE);
  MQ_REQUIRE(tensor || err, MQ_ERR_WORKSPACE, "mq_gptq_sweep: workspace too small");
  Engine eng(math, split, ws, st);
  // Tensor path: the factor is cut into transposed planes once (row n, k -> U[k][n]); the lazy
  // update of tile i1 then reads the window k in [i1, i1+128), rows n >= i2 of those planes,
  // and the sweep kernel writes its errors as planes itself.  No per-tile conversion passes.
  PlaneSet err_set, u_set;
  if (tensor) {
    MQ_REQUIRE(split >= 1 && split <= 3, MQ_ERR_ARGUMENT, "mq_gptq_sweep: split must be 1, 2 or 3 (got %d)", split);
    uint16_t* ep = ws.take<uint16_t>(plane_set_bytes(R, SUPER, split) / 2);
    uint16_t* up = ws.take<uint16_t>(plane_set_bytes(C, C, split) / 2);
    MQ_REQUIRE(ep && up, MQ_ERR_WORKSPACE, "mq_gptq_sweep: workspace too small for the operand planes");
    err_set.base = ep; err_set.planes = split; err_set.rows_pad = (int)pad_rows(R); err_set.total_rows = err_set.rows_pad;
    err_set.K_pad = SUPER;
    // the lazy updates read Uhat[i1:i2, i2:]: only blocks strictly above the diagonal
    MQ_TRY(make_planes_f32(Uhat, 1, ldu, (int)C, (int)C, split, up, &u_set, st, true, col_div));
  }
  SweepArgs sa;
  sa.W = W; sa.ldw = ldw; sa.R = (int)R;
  sa.U = Uhat; sa.ldu = ldu;
  sa.scale = scale; sa.zero = zero; sa.group = group; sa.s_rs = s_rs; sa.s_gs = s_gs;
  sa.maxq = (float)((1 << bits) - 1);
  sa.zero_default = 0.5f * (float)(1 << bits);
  sa.codes = codes; sa.C = C;
  sa.packed = packed;
  sa.deq = deq; sa.err = err;
  sa.Worig = Worig; sa.ldwo = ldwo;
  sa.err_planes = nullptr;
  sa.plane_stride = tensor ? err_set.total_rows * (int64_t)SUPER : 0;
  sa.n_planes = split;
  sa.err_ld = tensor ? SUPER : TILE;
  sa.bits = bits;
  // sixteen lanes per row while the grid holds every row group at once, eight beyond that
  const int lanes = ceil_div(R, TILE_THREADS / 16) <= MAX_SWEEP_CTAS ? 16 : 8;
  const bool uniform = group % (TILE / lanes) == 0;
  // every CTA stages the tile of the factor once and then walks row groups: no more CTAs than
  // two per SM, so that a tall layer does not stage the same tile thousands of times
  const int64_t row_groups = ceil_div(R, TILE_THREADS / lanes);
  const int grid = (int)(row_groups < MAX_SWEEP_CTAS ? row_groups : MAX_SWEEP_CTAS);
  // compact launches: full tiles whose groups are 32, 64 or a multiple of 128 columns wide run one
  // row per thread (a third slower per tile, on an eighth of the SMs)
  const int gpt = !compact ? 0 : group % TILE == 0 ? 1 : group == 64 ? 2 : group == 32 ? 4 : 0;

  for (int64_t i1 = 0; i1 < C; i1 += TILE) {
    const int nb = (int)((C - i1) < TILE ? (C - i1) : TILE);
    {
      // The kernel stages its tile of the factor before it waits for its predecessor: only a launch
      // that follows this loop's own update (which writes W, never the factor) may be chained.
      const bool chained = i1 > 0;
      // bytes the tile must move: W in, codes out, errors out, the triangle of Uhat once
      ProfScope prof(PROF_SWEEP_TILE, (double)R * nb * (4.0 + 1.0 + 4.0) + 2.0 * nb * nb, (double)R * nb * (nb - 1), st);
      sa.i1 = (int)i1; sa.nb = nb;
      if (tensor) sa.err_planes = err_set.base + (i1 % SUPER);
      if (gpt && nb == TILE) {
        switch (out_dtype) {
          case MQ_F32: MQ_TRY(launch_sweep_rows<MQ_F32>(chained, gpt, (int)R, st, sa)); break;
          case MQ_BF16: MQ_TRY(launch_sweep_rows<MQ_BF16>(chained, gpt, (int)R, st, sa)); break;
          default: MQ_TRY(launch_sweep_rows<MQ_F16>(chained, gpt, (int)R, st, sa));
        }
      } else {
        switch (out_dtype) {
          case MQ_F32: MQ_TRY(launch_sweep_tile<MQ_F32>(chained, uniform, lanes, grid, st, sa)); break;
          case MQ_BF16: MQ_TRY(launch_sweep_tile<MQ_BF16>(chained, uniform, lanes, grid, st, sa)); break;
          default: MQ_TRY(launch_sweep_tile<MQ_F16>(chained, uniform, lanes, grid, st, sa));
        }
      }
    }
    MQ_LAUNCH_CHECK();
    const int64_t i2 = i1 + nb;
    if (i2 >= C) break;
    if (!tensor) {
      GemmDesc g;
      g.A = err; g.a_rs = TILE; g.a_cs = 1;
      g.B = Uhat + i1 * ldu + i2; g.b_rs = ldu; g.b_cs = 1;
      g.C = W + i2; g.ldc = ldw;
      g.M = (int)R; g.N = (int)(C - i2); g.K = nb;
      g.alpha = 1.0f; g.beta = 1.0f;
      MQ_TRY(eng.gemm(g));
      continue;
    }
    const int64_t s0 = i1 / SUPER * SUPER;                        // first column of this super-block
    const int64_t s1 = (s0 + SUPER) < C ? (s0 + SUPER) : C;       // one past its last column
    if (i2 < s1) {
      // near: W[:, i2:s1] += E_tile Uhat[i1:i2, i2:s1]
      GemmDesc g;
      g.C = W + i2; g.ldc = ldw;
      g.M = (int)R; g.N = (int)(s1 - i2); g.K = nb;
      g.alpha = 1.0f; g.beta = 1.0f;
      g.compact = compact ? 1 : 0;
      PlaneSet a = err_set, b = u_set;
      a.k0 = (int)(i1 - s0);
      b.row0 = i2; b.k0 = (int)i1;
      MQ_TRY(gemm_tensor_planes(g, a, b, st));
    } else {
      // far: W[:, s1:] += E_super Uhat[s0:s1, s1:], all errors of the super-block in one contraction
      GemmDesc g;
      g.C = W + s1; g.ldc = ldw;
      g.M = (int)R; g.N = (int)(C - s1); g.K = (int)(s1 - s0);
      g.alpha = 1.0f; g.beta = 1.0f;
      PlaneSet b = u_set;
      b.row0 = s1; b.k0 = (int)s0;
      MQ_TRY(gemm_tensor_planes(g, err_set, b, st));
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
                             int64_t group_stride, int bits, int out_dtype, uint8_t* codes, int32_t* packed, void* dequantized,
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
  MQ_REQUIRE((math & ~MQ_MATH_COMPACT) == MQ_MATH_FP32 || (math & ~MQ_MATH_COMPACT) == MQ_MATH_TENSOR, MQ_ERR_ARGUMENT,
             "mq_gptq_sweep: bad math %d", math);
  Workspace ws(workspace, workspace_bytes);
  if (W_original) {
    MQ_REQUIRE(ldwo >= C && ldwo % 4 == 0 && aligned(W_original, 16) && W_original != W, MQ_ERR_ALIGNMENT,
               "mq_gptq_sweep: W_original must be a separate 16-byte aligned matrix with ldwo %% 4 == 0");
  }
  MQ_REQUIRE(!packed || (bits == 4 && !zero && aligned(packed, 4)), MQ_ERR_UNSUPPORTED,
             "mq_gptq_sweep: packed words need bits == 4, the symmetric zero point and a 4-byte aligned buffer");
  return gptq_sweep(W, R, C, ldw, Uhat, ldu, scale, zero, group, row_stride, group_stride, bits, out_dtype, codes,
                    dequantized, W_original, ldwo, math, split, ws, static_cast<cudaStream_t>(stream), nullptr, packed);
}
