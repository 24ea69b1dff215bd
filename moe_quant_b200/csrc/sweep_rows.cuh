// The row-per-thread sweep kernel for full tiles (included by sweep.cu).
#pragma once

#include "sweep.cuh"

namespace mq {

namespace {

// A full 128-column tile whose quantization groups are 32, 64 or a multiple of 128 columns wide.
// Each thread owns one weight row.  The row's 128 running weights live in shared memory, column
// major ([column][thread]: a warp's accesses are consecutive words), and pass through registers
// sixteen columns at a time:
//   chain:  the sixteen columns of chunk c, in order: quantize column j, add e_j U[j, k] to the
//           columns k behind it inside the chunk.  The only serial dependence is
//           quantize(j) -> one FMA -> quantize(j + 1).
//   spread: every later chunk takes the sixteen errors, e_t U[16c + t, k] for t = 0..15 in that
//           order: sixteen independent FMA chains per chunk, which fill the issue slots.
// The factor's row is read from shared memory at one address for the whole warp (a broadcast).
// Per element the operations and their order are those of the lane-per-chunk kernel: the codes
// are the same bit for bit.  A warp-instruction here advances 32 rows where that kernel advances
// 4, so a 2048-row layer needs 64 warps on 16 SMs for a few microseconds, which leaves the other
// SMs to the GEMMs of layers quantized next to it on other streams.  The loops over chunks are
// not unrolled: unrolled completely (weights in registers throughout) the 150 KB of straight-line
// code ran at the speed of instruction fetch, twice as slow as the kernel it was to replace.
constexpr int CHUNK = 16;
constexpr int N_CHUNKS = SWEEP_TILE / CHUNK;

template <int THREADS, int RPT>
constexpr size_t rows_smem_bytes() {
  return (size_t)(SWEEP_TILE * SWEEP_TILE + SWEEP_TILE * THREADS * RPT) * sizeof(float);   // factor tile + the rows' weights
}

// GPT: quantization groups per tile (1, 2 or 4); THREADS per CTA; RPT rows per thread
template <int DT, int GPT, int THREADS, int RPT>
__global__ void __launch_bounds__(THREADS, 1) sweep_rows_kernel(const SweepArgs a) {
  using T = typename StorageOf<DT>::type;
  constexpr int TILE = SWEEP_TILE;
  constexpr int CTA_ROWS = THREADS * RPT;
  extern __shared__ __align__(16) float rows_smem[];
  float* ublk = rows_smem;                 // [TILE][TILE]; only quads that reach past the diagonal are staged
  float* wS = rows_smem + TILE * TILE;     // [TILE][CTA_ROWS]
  const int i1 = a.i1, tid = threadIdx.x;
  {
    const float* src = a.U + (int64_t)i1 * a.ldu + i1;
    for (int idx = tid; idx < TILE * TILE / 4; idx += THREADS) {
      const int j = idx >> 5, k4 = (idx & 31) * 4;
      if (k4 + 3 > j) {
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&ublk[j * TILE + k4]);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + (int64_t)j * a.ldu + k4) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  chain_wait();
  chain_release();

  const float maxq = a.maxq;
  const bool inverse_free = a.Worig != nullptr;
  constexpr int GCOLS = TILE / GPT;
  bool staged = false;
  for (int row0 = blockIdx.x * CTA_ROWS; row0 < a.R; row0 += gridDim.x * CTA_ROWS) {
    bool valid[RPT];
    int r[RPT];
    const float* worow[RPT];
    float sc[RPT][GPT], zr[RPT][GPT], rs[RPT][GPT];
    float wo[RPT][CHUNK];
#pragma unroll
    for (int rr = 0; rr < RPT; ++rr) {
      valid[rr] = row0 + rr * THREADS + tid < a.R;
      r[rr] = valid[rr] ? row0 + rr * THREADS + tid : a.R - 1;   // rows past R repeat the last row and store nothing
      const float* wrow = a.W + (int64_t)r[rr] * a.ldw + i1;
      worow[rr] = inverse_free ? a.Worig + (int64_t)r[rr] * a.ldwo + i1 : wrow;
      float* wcol = wS + rr * THREADS + tid;                     // this row's weights: wcol[k * CTA_ROWS]
#pragma unroll 4
      for (int qd = 0; qd < TILE / 4; ++qd) {
        const float4 v = *reinterpret_cast<const float4*>(wrow + 4 * qd);
        wcol[(4 * qd) * CTA_ROWS] = v.x; wcol[(4 * qd + 1) * CTA_ROWS] = v.y;
        wcol[(4 * qd + 2) * CTA_ROWS] = v.z; wcol[(4 * qd + 3) * CTA_ROWS] = v.w;
      }
#pragma unroll
      for (int g = 0; g < GPT; ++g) {
        const int64_t off = (int64_t)r[rr] * a.s_rs + (int64_t)((i1 + g * GCOLS) / a.group) * a.s_gs;
        sc[rr][g] = __ldg(a.scale + off);
        zr[rr][g] = a.zero ? __ldg(a.zero + off) : a.zero_default;
        rs[rr][g] = 1.0f / sc[rr][g];
      }
#pragma unroll
      for (int qd = 0; qd < CHUNK / 4; ++qd) {
        const float4 v = *reinterpret_cast<const float4*>(worow[rr] + 4 * qd);
        wo[rr][4 * qd] = v.x; wo[rr][4 * qd + 1] = v.y; wo[rr][4 * qd + 2] = v.z; wo[rr][4 * qd + 3] = v.w;
      }
    }
    if (!staged) {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncthreads();
      staged = true;
    }
    float* wmine = wS + tid;

#pragma unroll 1
    for (int c = 0; c < N_CHUNKS; ++c) {
      const int j0 = c * CHUNK;
      const int gi = j0 / GCOLS;   // a chunk lies in one group
      float s_t[RPT], z_t[RPT], r_t[RPT];
#pragma unroll
      for (int rr = 0; rr < RPT; ++rr) {
        s_t[rr] = sc[rr][0]; z_t[rr] = zr[rr][0]; r_t[rr] = rs[rr][0];
        if constexpr (GPT > 1) {
          if (gi == 1) { s_t[rr] = sc[rr][1]; z_t[rr] = zr[rr][1]; r_t[rr] = rs[rr][1]; }
        }
        if constexpr (GPT > 2) {
          if (gi == 2) { s_t[rr] = sc[rr][2]; z_t[rr] = zr[rr][2]; r_t[rr] = rs[rr][2]; }
          if (gi == 3) { s_t[rr] = sc[rr][3]; z_t[rr] = zr[rr][3]; r_t[rr] = rs[rr][3]; }
        }
      }
      float w[RPT][CHUNK], e[RPT][CHUNK], y16[RPT][CHUNK];
      uint32_t cw[RPT][4];
#pragma unroll
      for (int rr = 0; rr < RPT; ++rr)
#pragma unroll
        for (int t = 0; t < CHUNK; ++t) w[rr][t] = wmine[(j0 + t) * CTA_ROWS + rr * THREADS];
      // ---- chain (the rows of a thread are independent: their chains interleave)
      const float* ud = ublk + j0 * TILE + j0;   // the chunk's own 16 x 16 block of the factor
#pragma unroll
      for (int t = 0; t < CHUNK; ++t) {
        float4 ur[CHUNK / 4];
#pragma unroll
        for (int qd = t >> 2; qd < CHUNK / 4; ++qd) {
          if (qd == (t >> 2) && (t & 3) == 3) continue;
          ur[qd] = *reinterpret_cast<const float4*>(ud + t * TILE + 4 * qd);
        }
#pragma unroll
        for (int rr = 0; rr < RPT; ++rr) {
          const float x = w[rr][t];
          float d = x * r_t[rr];
          d = fmaf(fmaf(-s_t[rr], d, x), r_t[rr], d);
          const float q = fminf(fmaxf(floorf((d + z_t[rr]) + 0.5f), 0.0f), maxq);
          const float y = round_through<DT>((q - z_t[rr]) * s_t[rr]);
          const float et = inverse_free ? (wo[rr][t] - y) : (y - x);
          e[rr][t] = et;
          y16[rr][t] = y;
          if ((t & 3) == 0) cw[rr][t >> 2] = (uint32_t)q;
          else cw[rr][t >> 2] |= (uint32_t)q << (8 * (t & 3));
          // the rest of t's own quad one by one, whole quads after it
          if ((t & 3) != 3) {
            const float4 u = ur[t >> 2];
            if ((t & 3) < 1) w[rr][(t & ~3) + 1] = fmaf(u.y, et, w[rr][(t & ~3) + 1]);
            if ((t & 3) < 2) w[rr][(t & ~3) + 2] = fmaf(u.z, et, w[rr][(t & ~3) + 2]);
            w[rr][(t & ~3) + 3] = fmaf(u.w, et, w[rr][(t & ~3) + 3]);
          }
          const float2 e2 = make_float2(et, et);
#pragma unroll
          for (int qd = (t >> 2) + 1; qd < CHUNK / 4; ++qd) {
            const float4 u = ur[qd];
            // packed fp32 FMA: two columns per instruction, each half an ordinary fma.rn
            const float2 p01 = __ffma2_rn(make_float2(u.x, u.y), e2, make_float2(w[rr][4 * qd], w[rr][4 * qd + 1]));
            const float2 p23 = __ffma2_rn(make_float2(u.z, u.w), e2, make_float2(w[rr][4 * qd + 2], w[rr][4 * qd + 3]));
            w[rr][4 * qd] = p01.x; w[rr][4 * qd + 1] = p01.y; w[rr][4 * qd + 2] = p23.x; w[rr][4 * qd + 3] = p23.y;
          }
        }
      }
      // the original weights of the next chunk are on their way while the errors spread
      if (c + 1 < N_CHUNKS) {
#pragma unroll
        for (int rr = 0; rr < RPT; ++rr)
#pragma unroll
          for (int qd = 0; qd < CHUNK / 4; ++qd) {
            const float4 v = *reinterpret_cast<const float4*>(worow[rr] + j0 + CHUNK + 4 * qd);
            wo[rr][4 * qd] = v.x; wo[rr][4 * qd + 1] = v.y; wo[rr][4 * qd + 2] = v.z; wo[rr][4 * qd + 3] = v.w;
          }
      }
      // ---- spread: the chunks behind take the sixteen errors, nearest first; a value of the
      // factor read from shared memory serves all the rows of the thread
#pragma unroll 1
      for (int kc = c + 1; kc < N_CHUNKS; ++kc) {
        float v[RPT][CHUNK];
        float* wk = wmine + (kc * CHUNK) * CTA_ROWS;
#pragma unroll
        for (int rr = 0; rr < RPT; ++rr)
#pragma unroll
          for (int k = 0; k < CHUNK; ++k) v[rr][k] = wk[k * CTA_ROWS + rr * THREADS];
        const float* uk = ublk + j0 * TILE + kc * CHUNK;
#pragma unroll
        for (int t = 0; t < CHUNK; ++t) {
#pragma unroll
          for (int qd = 0; qd < CHUNK / 4; ++qd) {
            const float4 u = *reinterpret_cast<const float4*>(uk + t * TILE + 4 * qd);
#pragma unroll
            for (int rr = 0; rr < RPT; ++rr) {
              const float2 e2 = make_float2(e[rr][t], e[rr][t]);
              const float2 p01 = __ffma2_rn(make_float2(u.x, u.y), e2, make_float2(v[rr][4 * qd], v[rr][4 * qd + 1]));
              const float2 p23 = __ffma2_rn(make_float2(u.z, u.w), e2, make_float2(v[rr][4 * qd + 2], v[rr][4 * qd + 3]));
              v[rr][4 * qd] = p01.x; v[rr][4 * qd + 1] = p01.y; v[rr][4 * qd + 2] = p23.x; v[rr][4 * qd + 3] = p23.y;
            }
          }
        }
#pragma unroll
        for (int rr = 0; rr < RPT; ++rr)
#pragma unroll
          for (int k = 0; k < CHUNK; ++k) wk[k * CTA_ROWS + rr * THREADS] = v[rr][k];
      }
      // ---- what the chunk produced
#pragma unroll
      for (int rr = 0; rr < RPT; ++rr) {
        if (!valid[rr]) continue;
        const int64_t row = r[rr];
        uint2* cdst = reinterpret_cast<uint2*>(a.codes + row * a.C + i1 + j0);
        cdst[0] = make_uint2(cw[rr][0], cw[rr][1]);
        cdst[1] = make_uint2(cw[rr][2], cw[rr][3]);
        if (a.packed) {
          int32_t* pdst = a.packed + row * (a.C >> 3) + ((i1 + j0) >> 3);
          pdst[0] = (int32_t)pack_nibbles(cw[rr][0], cw[rr][1]);
          pdst[1] = (int32_t)pack_nibbles(cw[rr][2], cw[rr][3]);
        }
        if (a.err_planes) {
          uint32_t hp[CHUNK / 2], mp[CHUNK / 2], lp[CHUNK / 2];
#pragma unroll
          for (int t = 0; t < CHUNK; t += 2) {
            uint16_t h0, m0, l0, h1, m1, l1;
            split_bf16x3(e[rr][t], h0, m0, l0);
            split_bf16x3(e[rr][t + 1], h1, m1, l1);
            hp[t >> 1] = (uint32_t)h0 | ((uint32_t)h1 << 16);
            mp[t >> 1] = (uint32_t)m0 | ((uint32_t)m1 << 16);
            lp[t >> 1] = (uint32_t)l0 | ((uint32_t)l1 << 16);
          }
          uint16_t* dst = a.err_planes + row * a.err_ld + j0;
          reinterpret_cast<uint4*>(dst)[0] = make_uint4(hp[0], hp[1], hp[2], hp[3]);
          reinterpret_cast<uint4*>(dst)[1] = make_uint4(hp[4], hp[5], hp[6], hp[7]);
          if (a.n_planes > 1) {
            reinterpret_cast<uint4*>(dst + a.plane_stride)[0] = make_uint4(mp[0], mp[1], mp[2], mp[3]);
            reinterpret_cast<uint4*>(dst + a.plane_stride)[1] = make_uint4(mp[4], mp[5], mp[6], mp[7]);
          }
          if (a.n_planes > 2) {
            reinterpret_cast<uint4*>(dst + 2 * a.plane_stride)[0] = make_uint4(lp[0], lp[1], lp[2], lp[3]);
            reinterpret_cast<uint4*>(dst + 2 * a.plane_stride)[1] = make_uint4(lp[4], lp[5], lp[6], lp[7]);
          }
        } else {
          float4* dst = reinterpret_cast<float4*>(a.err + row * a.err_ld + j0);
#pragma unroll
          for (int qd = 0; qd < CHUNK / 4; ++qd)
            dst[qd] = make_float4(e[rr][4 * qd], e[rr][4 * qd + 1], e[rr][4 * qd + 2], e[rr][4 * qd + 3]);
        }
        if (a.deq) {
          T* dq = static_cast<T*>(a.deq) + row * a.C + i1 + j0;
#pragma unroll
          for (int t = 0; t < CHUNK; ++t) dq[t] = from_float<T>(y16[rr][t]);
        }
      }
    }
  }
  if (!staged) asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// 64 threads x 1 row measured best (33 / 29 / 44 / 45 us per 2048-row tile for 128x1 / 64x1 / 32x2 /
// 64x2 threads x rows: two rows per thread double a warp's instruction stream for little more overlap).
constexpr int ROWS_THREADS = 64;
constexpr int ROWS_PER_THREAD = 1;

template <int DT, int GPT>
int launch_rows_gpt(bool chained, int R, cudaStream_t st, const SweepArgs& args) {
  constexpr size_t smem = rows_smem_bytes<ROWS_THREADS, ROWS_PER_THREAD>();
  static bool configured[64] = {};
  int dev = 0;
  MQ_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    MQ_CUDA(cudaFuncSetAttribute(sweep_rows_kernel<DT, GPT, ROWS_THREADS, ROWS_PER_THREAD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem));
    configured[dev & 63] = true;
  }
  const int ctas = (R + ROWS_THREADS * ROWS_PER_THREAD - 1) / (ROWS_THREADS * ROWS_PER_THREAD);
  MQ_CUDA(launch_chained(chained, sweep_rows_kernel<DT, GPT, ROWS_THREADS, ROWS_PER_THREAD>, dim3(ctas < 2 * 148 ? ctas : 2 * 148),
                         dim3(ROWS_THREADS), smem, st, args));
  return MQ_OK;
}

template <int DT>
int launch_sweep_rows(bool chained, int gpt, int R, cudaStream_t st, const SweepArgs& args) {
  if (gpt == 1) return launch_rows_gpt<DT, 1>(chained, R, st, args);
  if (gpt == 2) return launch_rows_gpt<DT, 2>(chained, R, st, args);
  return launch_rows_gpt<DT, 4>(chained, R, st, args);
}

}  // namespace

}  // namespace mq
