// tcgen05 tensor-core GEMM on bf16/fp16 planes: the MQ_MATH_TENSOR arithmetic.
//
//   C[m,n] = alpha * sum over terms (i,j) of  A_i[m,:] . B_j[n,:]  + beta * C[m,n]
//
// A_i / B_j are 16-bit "planes" of the operands, both stored K-major (the reduction
// index contiguous) so that a 128 x 64 tile is 128 rows of 128 bytes: exactly one TMA
// box with the 128-byte swizzle and exactly the canonical K-major shared-memory
// layout that tcgen05.mma reads through a matrix descriptor.  An fp32 operand x is cut
// into planes hi = bf16(x), mid = bf16(x - hi), lo = bf16(x - hi - mid); products of two
// bf16 numbers are exact in fp32, so keeping the terms with i + j < planes recovers
// fp32-grade products (planes = 3: six products, error ~2^-24) on the tensor pipe.
//
// Three kernels share the pieces below: umma_gemm_kernel (one tile per CTA, any K, planes,
// batches), umma_gemm_persistent_kernel (one-plane GEMMs and the Hessian: one CTA per SM walks
// 128 x 256 tiles, epilogue under the next tile's MMAs; 16-bit activations are read in place as
// MN-major boxes) and umma_panel_kernel (K <= 128, A stationary, C through the TMA unit).
// Structure of the first (one 128 x 128 output tile per CTA, 192 threads):
//   warp 0, one lane : TMA producer, fills a ring of shared-memory stages
//   warp 1, one lane : issues tcgen05.mma (M128 N128 K16) into a 128-column TMEM
//                      accumulator, releases stages with tcgen05.commit
//   warps 2..5       : epilogue, tcgen05.ld the accumulator (one TMEM lane = one output
//                      row per thread), alpha/beta, bounds, stores
// Every mbarrier wait is bounded; a wait that expires records a code in g_engine_fault,
// the kernel still frees its TMEM and returns.
#include <cuda.h>
#include <cstring>

#include "engine.cuh"
#include "profile.cuh"

namespace mq {

__device__ int g_engine_fault = 0;

namespace {

constexpr int TILE_M = 128, TILE_N = 128, SLAB_K = 64;
constexpr int PLANE_TILE_BYTES = TILE_M * SLAB_K * 2;  // 16 KB
constexpr int GEMM_THREADS = 192;
constexpr int STAGE_LD = 36;                        // floats per row of an epilogue staging tile
constexpr int STAGE_BYTES = 4 * 32 * STAGE_LD * 4;  // four epilogue warps

struct UmmaParams {
  float* C;
  int64_t ldc, c_bs;
  int M, N, K;
  float alpha, beta;
  int upper_tiles_only, a_upper, b_upper;
  int n_total, n_step, k_follows_n;
  int a_rows_pad, b_rows_pad;  // rows each batch occupies in the stacked plane buffers
  int a_row0, a_k0, b_row0, b_k0;  // origin of the operand windows inside their plane buffers
  int planes, nterms, stages;
  uint32_t idesc;
  int mirror;  // symmetric result: every block above the diagonal is also stored transposed
  int c_tma;   // panel kernel epilogue: 0 = loads/stores by the warps, 1 = TMA store (beta == 0), 2 = TMA add (beta == 1)
  int drain_slabs;  // streaming kernel: slabs of k per accumulator before it is added to C (0 = all of K)
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait: gives up after about one second and records `code`.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 255u) == 255u) {
      // once any wait on this device has expired, every later wait gives up at once
      if (*reinterpret_cast<volatile int*>(&g_engine_fault) != 0) return false;
      uint64_t now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > 1000000000ull) {
        atomicCAS(&g_engine_fault, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Epilogue through the TMA unit: a 32 x 32 fp32 box leaves shared memory as one bulk tensor
// store, or as an element-wise fp32 add performed at the L2 (C += box) so that the SM never
// reads C.  Completion is tracked with bulk async-groups of the issuing thread.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Matrix descriptor of a K-major tile with the 128-byte swizzle: rows of 128 bytes,
// groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset: unused with a swizzle
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;            // version
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}

// Matrix descriptor of an MN-major operand with the 128-byte swizzle, as a TMA box of
// 64 (m or n, contiguous) x 64 (k) 16-bit elements lands in shared memory: one 128-byte row per
// k, groups of 8 k 1024 bytes apart (stride byte offset), 64-wide blocks of m/n `block_bytes`
// apart (leading byte offset).
__device__ __forceinline__ uint64_t mnmajor_sw128_desc(uint32_t smem_addr, uint32_t block_bytes) {
  uint64_t d = (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(block_bytes >> 4) << 16;  // leading byte offset
  d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset
  d |= (uint64_t)1 << 46;                   // version
  d |= (uint64_t)2 << 61;                   // SWIZZLE_128B
  return d;
}

// One 64-wide K slab of a one-plane GEMM whose operands are MN-major boxes (8 KB per 64 rows of
// m/n): a K step of 16 is two groups of 8 k, 2048 bytes.
__device__ __forceinline__ void issue_slab_mn(uint32_t tmem_d, uint32_t a_tile, uint32_t b_tile, uint32_t idesc,
                                              uint32_t& accumulate) {
  const uint64_t a0 = mnmajor_sw128_desc(a_tile, 8192), b0 = mnmajor_sw128_desc(b_tile, 8192);
#pragma unroll
  for (int kk = 0; kk < SLAB_K / 16; ++kk) {
    umma_bf16(tmem_d, a0 + (uint64_t)((kk * 2048) >> 4), b0 + (uint64_t)((kk * 2048) >> 4), idesc, accumulate);
    accumulate = 1;
  }
}

// All MMAs of one 64-wide K slab: for each of the four K16 steps, the products A_i B_j with
// i + j < PLANES.  The issuing thread must feed the tensor pipe one MMA every ~64 cycles, so
// the loops are unrolled at compile time and a descriptor costs one 32-bit add: only the
// address field (low word) changes between tiles, planes and K steps.
// The leading product (hi x hi) and the correction products go to two different accumulators,
// `tmem_d` and `tmem_d + small_off`, which the epilogue adds in fp32.  The corrections are 2^-8 and
// 2^-16 of the leading term: summed into one accumulator they would each cost it a rounding at
// full magnitude (48 roundings per 128 of k instead of 8), and the tensor core's accumulation
// does not round to nearest; kept apart, the small sums keep their own low bits.
template <int PLANES>
__device__ __forceinline__ void issue_slab(uint32_t tmem_d, uint32_t small_off, uint32_t a_tile, uint32_t b_tile, uint32_t idesc,
                                           uint32_t& accumulate, uint32_t& accumulate_small) {
  const uint64_t a0 = kmajor_sw128_desc(a_tile), b0 = kmajor_sw128_desc(b_tile);
  const uint32_t hi = (uint32_t)(a0 >> 32);
  const uint32_t a_lo = (uint32_t)a0, b_lo = (uint32_t)b0;
#pragma unroll
  for (int kk = 0; kk < SLAB_K / 16; ++kk) {
#pragma unroll
    for (int ti = 0; ti < PLANES; ++ti) {
#pragma unroll
      for (int tj = 0; tj < PLANES; ++tj) {
        if (ti + tj < PLANES) {
          const uint64_t ad = ((uint64_t)hi << 32) | (uint64_t)(a_lo + (uint32_t)((ti * PLANE_TILE_BYTES + kk * 32) >> 4));
          const uint64_t bd = ((uint64_t)hi << 32) | (uint64_t)(b_lo + (uint32_t)((tj * PLANE_TILE_BYTES + kk * 32) >> 4));
          if (ti + tj == 0) {
            umma_bf16(tmem_d, ad, bd, idesc, accumulate);
            accumulate = 1;
          } else {
            umma_bf16(tmem_d + small_off, ad, bd, idesc, accumulate_small);
            accumulate_small = 1;
          }
        }
      }
    }
  }
}

__device__ __forceinline__ void issue_slab_any(int planes, uint32_t tmem_d, uint32_t small_off, uint32_t a_tile, uint32_t b_tile,
                                               uint32_t idesc, uint32_t& accumulate, uint32_t& accumulate_small) {
  if (planes == 3) issue_slab<3>(tmem_d, small_off, a_tile, b_tile, idesc, accumulate, accumulate_small);
  else if (planes == 2) issue_slab<2>(tmem_d, small_off, a_tile, b_tile, idesc, accumulate, accumulate_small);
  else issue_slab<1>(tmem_d, small_off, a_tile, b_tile, idesc, accumulate, accumulate_small);
}

// 32 accumulator columns of this warp's TMEM lanes; with small_off != 0 the sum of the leading
// and the correction accumulator.
__device__ __forceinline__ void tmem_ld32_sum(uint32_t taddr, uint32_t small_off, float (&v)[32]) {
  tmem_ld32(taddr, v);
  if (small_off) {
    float c[32];
    tmem_ld32(taddr + small_off, c);
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] += c[i];
  }
}

// Epilogue of one 128 x TN tile by the four epilogue warps: C <- alpha * acc + beta * C with the
// symmetric-result handling described inside.  `stage_base` is 4 x 32 x STAGE_LD floats of
// shared memory; the accumulator is waited for on (acc_bar, acc_parity) after the first half of
// C has been requested.  Returns false when that wait expired.
template <int TN>
__device__ __forceinline__ bool epilogue_tile(const float alpha, const float beta, const int64_t ldc, const int M, const int mirror,
                                              float* __restrict__ C, const int m0, const int n0,
                                              const int N, const uint32_t tmem_acc, float* stage_base, const int warp,
                                              const int lane, const bool have_acc, const uint32_t acc_bar,
                                              const uint32_t acc_parity, const uint32_t small_off = 0) {
  const int q = warp & 3;  // TMEM lane quadrant this warp may read
  const int row = m0 + q * 32 + lane;
  const bool vec_ok = (ldc & 3) == 0 && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
  // whole 32 x TN quadrant in range: coalesced path (uniform in the warp, tcgen05.ld is warp-wide)
  const bool whole = vec_ok && m0 + q * 32 + 32 <= M && n0 + TN <= N;
  bool ok = true;
  bool waited = false;
  if (whole) {
    // lane l handles row 4*it + l/8, columns 4*(l%8).. of each 32-column chunk: every global
    // access of the warp is four full 128-byte row segments.  The first 128 columns of C are
    // requested before the accumulator is waited for.
    float* cq = C + (int64_t)(m0 + q * 32 + (lane >> 3)) * ldc + n0 + (lane & 7) * 4;
    // Symmetric result (mirror): the upper triangle is authoritative.  In units of 32 x 32
    // blocks (gr, gc): gc > gr is stored and also stored transposed, gc == gr is symmetrised
    // (A_i B_j and A_j B_i are summed in different orders by the MMA), gc < gr is left to the
    // transposed store of its mirror block.  C[n,m] == C[m,n] then holds bit for bit.
    const int gr = (m0 >> 5) + q;
#pragma unroll 1
    for (int half = 0; half < TN / 128 && ok; ++half) {
      float4 old[32];
      if (beta != 0.0f) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int it = 0; it < 8; ++it)
            old[c * 8 + it] = *reinterpret_cast<const float4*>(cq + (int64_t)(4 * it) * ldc + half * 128 + c * 32);
      }
      if (!waited) {
        if (have_acc) ok = mbar_wait(acc_bar, acc_parity, 3);
        tc_fence_after();
        waited = true;
        if (!ok) break;
      }
      float* stage = stage_base + (warp - 2) * 32 * STAGE_LD;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v[32];
        if (have_acc) {
          tmem_ld32_sum(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * 128 + c * 32), small_off, v);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.0f;
        }
        const int gc = ((n0 + half * 128) >> 5) + c;
        const bool store_direct = !mirror || gc > gr;
        const bool store_mirror = mirror && gc > gr;
        const bool symmetrise = mirror && gc == gr;
        const int coff = half * 128 + c * 32;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(&stage[lane * STAGE_LD + 4 * j]) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          float* sp = &stage[(4 * it + (lane >> 3)) * STAGE_LD + (lane & 7) * 4];
          const float4 a4 = *reinterpret_cast<const float4*>(sp);
          float4 o = make_float4(alpha * a4.x, alpha * a4.y, alpha * a4.z, alpha * a4.w);
          if (beta != 0.0f) {
            const float4 od = old[c * 8 + it];
            o.x = fmaf(beta, od.x, o.x); o.y = fmaf(beta, od.y, o.y);
            o.z = fmaf(beta, od.z, o.z); o.w = fmaf(beta, od.w, o.w);
          }
          if (store_direct) *reinterpret_cast<float4*>(cq + (int64_t)(4 * it) * ldc + coff) = o;
          if (mirror) *reinterpret_cast<float4*>(sp) = o;  // keep the final values for the stores below
        }
        __syncwarp();
        if (symmetrise) {
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = 4 * it + (lane >> 3), cc = (lane & 7) * 4;
            float e[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) e[t] = (cc + t >= r) ? stage[r * STAGE_LD + cc + t] : stage[(cc + t) * STAGE_LD + r];
            *reinterpret_cast<float4*>(cq + (int64_t)(4 * it) * ldc + coff) = make_float4(e[0], e[1], e[2], e[3]);
          }
        }
        if (store_mirror) {
          // C[n0 + coff + i][m0 + 32q + l] = final[l][i]: one 128-byte row segment per i
          float* mq = C + (int64_t)(n0 + coff) * ldc + m0 + q * 32 + lane;
#pragma unroll 8
          for (int i = 0; i < 32; ++i) mq[(int64_t)i * ldc] = stage[lane * STAGE_LD + i];
        }
        __syncwarp();
      }
    }
  } else {
    if (have_acc) ok = mbar_wait(acc_bar, acc_parity, 3);
    tc_fence_after();
    if (ok) {
#pragma unroll 1
      for (int c = 0; c < TN / 32; ++c) {
        float v[32];
        if (have_acc) {
          tmem_ld32_sum(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), small_off, v);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.0f;
        }
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
          float* dst = C + (int64_t)row * ldc + col0;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col0 + j < N) {
              float o = alpha * v[j];
              if (beta != 0.0f) o = fmaf(beta, dst[j], o);
              // symmetric result: the upper triangle is authoritative; inside a diagonal 32 x 32
              // block the coalesced path symmetrises, so take the element of the upper half there too
              if (!(mirror && col0 + j < row)) dst[j] = o;
              if (mirror && col0 + j > row) C[(int64_t)(col0 + j) * ldc + row] = o;
            }
          }
        }
      }
    }
  }
  return ok;
}

// ---------------------------------------------------------------- the GEMM kernel
// One 128 x TN tile per CTA, any number of planes, batches, triangular k-ranges.  Instantiated
// with TN = 128; one-plane GEMMs with N >= 256 go to umma_gemm_persistent_kernel (256-wide tiles
// halve the A bytes streamed per flop, which is what limits a one-product GEMM).
template <int TN>
__global__ void __launch_bounds__(GEMM_THREADS) umma_gemm_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                 const __grid_constant__ CUtensorMap map_b,
                                                                 const UmmaParams p) {
  constexpr int B_TILE_BYTES = TN * SLAB_K * 2;
  const int b = blockIdx.z;
  const int m0 = blockIdx.y * TILE_M, n0 = blockIdx.x * TN;
  int N = p.N, K = p.K;
  if (p.n_step) {
    int left = p.n_total - b * p.n_step;
    N = N < left ? N : left;
    if (p.k_follows_n) K = N;
  }
  if (N <= 0 || n0 >= N || m0 >= p.M) return;
  if (p.upper_tiles_only && n0 + TN <= m0) return;
  const int k_lo = p.a_upper ? (m0 / SLAB_K) * SLAB_K : 0;
  int k_hi = K;
  if (p.b_upper && n0 + TN < k_hi) k_hi = n0 + TN;
  const int n_slabs = k_hi > k_lo ? (k_hi - k_lo + SLAB_K - 1) / SLAB_K : 0;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // the swizzle pattern repeats every 1024 bytes
  const int planes = p.planes;
  const uint32_t stage_bytes = (uint32_t)planes * (PLANE_TILE_BYTES + B_TILE_BYTES);
  __shared__ __align__(8) uint64_t bars[2 * 4 + 1];
  __shared__ uint32_t tmem_slot;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[4]), acc_bar = smem_u32(&bars[8]);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t idesc = p.idesc;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // with more than one plane the correction products get an accumulator of their own
  const uint32_t small_off = planes > 1 ? (uint32_t)TN : 0u;
  const uint32_t tmem_cols = planes > 1 ? 2 * TN : TN;
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const int a_row = b * p.a_rows_pad + m0 + p.a_row0, b_row = b * p.b_rows_pad + n0 + p.b_row0;
      for (int s = 0; s < n_slabs; ++s) {
        const int st = s % p.stages;
        if (s >= p.stages && !mbar_wait(empty0 + 8 * st, ((s / p.stages) - 1) & 1, 1)) break;
        mbar_expect_tx(full0 + 8 * st, stage_bytes);
        const uint32_t dst = smem_base + st * stage_bytes;
        const int k = k_lo + s * SLAB_K;
        for (int pl = 0; pl < planes; ++pl) {
          tma_load_3d(dst + pl * PLANE_TILE_BYTES, &map_a, full0 + 8 * st, k + p.a_k0, a_row, pl);
          const uint32_t bdst = dst + planes * PLANE_TILE_BYTES + pl * B_TILE_BYTES;
#pragma unroll
          for (int h = 0; h < TN / TILE_M; ++h)  // the TMA box is 128 rows
            tma_load_3d(bdst + h * PLANE_TILE_BYTES, &map_b, full0 + 8 * st, k + p.b_k0, b_row + h * TILE_M, pl);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t accumulate = 0, accumulate_small = 0;
      bool ok = true;
      for (int s = 0; s < n_slabs && ok; ++s) {
        const int st = s % p.stages;
        ok = mbar_wait(full0 + 8 * st, (s / p.stages) & 1, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_base = smem_base + st * stage_bytes;
        const uint32_t b_base = a_base + planes * PLANE_TILE_BYTES;
        if (TN == 128) issue_slab_any(planes, tmem_acc, small_off, a_base, b_base, idesc, accumulate, accumulate_small);
        else issue_slab<1>(tmem_acc, 0u, a_base, b_base, idesc, accumulate, accumulate_small);
        umma_commit(empty0 + 8 * st);  // the stage is free once these MMAs have read it
      }
      umma_commit(acc_bar);  // arrives when every MMA issued above has completed
    }
  } else {
    // every MMA has completed when the accumulator barrier fires, so the operand stages are
    // free: stage 0 becomes the staging tiles
    epilogue_tile<TN>(p.alpha, p.beta, p.ldc, p.M, p.mirror, p.C + (int64_t)b * p.c_bs, m0, n0, N, tmem_acc,
                      reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw))), warp, lane, n_slabs > 0, acc_bar, 0,
                      small_off);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, tmem_cols);
  }
}

// ---------------------------------------------------------------- persistent one-plane GEMM (the Hessian)
// 128 x 256 tiles, one plane per operand (bf16/fp16 activations), any K.  One CTA per SM walks the
// list of kept tiles (index = blockIdx.x + i * gridDim.x): the operand ring keeps running across
// tiles, the accumulator alternates between the two halves of tensor memory, and the epilogue of
// tile i (read-modify-write of C and, for the symmetric Hessian, the transposed store) runs while
// tile i+1 is multiplied.  With one tile per CTA the tensor pipe idled through every prologue and
// epilogue.
constexpr int PERSIST_TN = 256, PERSIST_STAGES = 4;

// kept tile number w -> tile row ty, tile column tx (row-major over the kept tiles)
__device__ __forceinline__ void persistent_tile(const UmmaParams& p, int w, int nx_tiles, int& ty, int& tx) {
  if (!p.upper_tiles_only) {
    ty = w / nx_tiles;
    tx = w - ty * nx_tiles;
    return;
  }
  ty = 0;
  for (;;) {
    const int tx0 = (ty * TILE_M) / PERSIST_TN;  // first tile of the row that reaches the diagonal
    const int cnt = nx_tiles - tx0;
    if (w < cnt) { tx = tx0 + w; return; }
    w -= cnt;
    ++ty;
  }
}

// DIRECT: the operands are not plane buffers but one row-major 16-bit matrix X (k x m, the
// activations: tokens x channels) read in place through a 2-D map (map_a; map_b unused) with
// 64 x 64 boxes, which arrive MN-major; C <- alpha X^T X + beta C.
template <bool DIRECT>
__global__ void __launch_bounds__(GEMM_THREADS, 1) umma_gemm_persistent_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                            const __grid_constant__ CUtensorMap map_b,
                                                                            const UmmaParams p, const int n_work) {
  constexpr int TN = PERSIST_TN, NST = PERSIST_STAGES;
  constexpr uint32_t STAGE = PLANE_TILE_BYTES + TN * SLAB_K * 2;  // A 16 KB + B 32 KB
  const int nx_tiles = (p.N + TN - 1) / TN;
  const int n_slabs = (p.K + SLAB_K - 1) / SLAB_K;
  const int my_tiles = ((int)blockIdx.x < n_work) ? (n_work - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  if (my_tiles == 0) return;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ __align__(8) uint64_t bars[2 * NST + 4];
  __shared__ uint32_t tmem_slot;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[NST]);
  const uint32_t acc_full = smem_u32(&bars[2 * NST]), acc_empty = smem_u32(&bars[2 * NST + 2]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(acc_full + 8 * s, 1);
      mbar_init(acc_empty + 8 * s, 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), 2 * TN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = tmem_slot;

  if (warp == 0) {
    int it = 0;
    bool ok = true;
    for (int i = 0; i < my_tiles && ok; ++i) {
      int ty, tx;
      persistent_tile(p, (int)blockIdx.x + i * (int)gridDim.x, nx_tiles, ty, tx);
      const int a_row = ty * TILE_M + p.a_row0, b_row = tx * TN + p.b_row0;
      for (int s = 0; s < n_slabs; ++s, ++it) {
        const int st = it % NST;
        if (it >= NST && !mbar_wait(empty0 + 8 * st, ((it / NST) - 1) & 1, 31)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(full0 + 8 * st, STAGE);
          const uint32_t dst = smem_base + (uint32_t)st * STAGE;
          if (DIRECT) {
            // boxes of 64 channels x 64 tokens, 8 KB each: two for A, four for B
#pragma unroll
            for (int h = 0; h < TILE_M / 64; ++h) tma_load_2d(dst + h * 8192, &map_a, full0 + 8 * st, a_row + h * 64, s * SLAB_K);
#pragma unroll
            for (int h = 0; h < TN / 64; ++h)
              tma_load_2d(dst + PLANE_TILE_BYTES + h * 8192, &map_a, full0 + 8 * st, b_row + h * 64, s * SLAB_K);
          } else {
            tma_load_3d(dst, &map_a, full0 + 8 * st, s * SLAB_K + p.a_k0, a_row, 0);
#pragma unroll
            for (int h = 0; h < TN / TILE_M; ++h)  // the TMA box is 128 rows
              tma_load_3d(dst + PLANE_TILE_BYTES + h * PLANE_TILE_BYTES, &map_b, full0 + 8 * st, s * SLAB_K + p.b_k0,
                          b_row + h * TILE_M, 0);
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    int it = 0;
    bool ok = true;
    for (int i = 0; i < my_tiles && ok; ++i) {
      const int acc = i & 1;
      if (i >= 2) ok = mbar_wait(acc_empty + 8 * acc, ((i >> 1) - 1) & 1, 32);
      if (!ok) break;
      tc_fence_after();
      uint32_t accumulate = 0, unused_small = 0;
      for (int s = 0; s < n_slabs && ok; ++s, ++it) {
        const int st = it % NST;
        ok = mbar_wait(full0 + 8 * st, (it / NST) & 1, 33);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_base = smem_base + (uint32_t)st * STAGE;
          if (DIRECT) issue_slab_mn(tmem_acc + (uint32_t)(acc * TN), a_base, a_base + PLANE_TILE_BYTES, p.idesc, accumulate);
          else issue_slab<1>(tmem_acc + (uint32_t)(acc * TN), 0u, a_base, a_base + PLANE_TILE_BYTES, p.idesc, accumulate, unused_small);
          umma_commit(empty0 + 8 * st);
        }
        __syncwarp();
      }
      if (ok && lane == 0) umma_commit(acc_full + 8 * acc);
      __syncwarp();
    }
  } else {
    float* stage_base = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)) + (uint32_t)NST * STAGE);
    bool ok = true;
    for (int i = 0; i < my_tiles && ok; ++i) {
      const int acc = i & 1;
      int ty, tx;
      persistent_tile(p, (int)blockIdx.x + i * (int)gridDim.x, nx_tiles, ty, tx);
      ok = epilogue_tile<TN>(p.alpha, p.beta, p.ldc, p.M, p.mirror, p.C, ty * TILE_M, tx * TN, p.N, tmem_acc + (uint32_t)(acc * TN), stage_base, warp, lane,
                             n_slabs > 0, acc_full + 8 * acc, (uint32_t)((i >> 1) & 1));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + 8 * acc);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, 2 * TN);
  }
}

// ---------------------------------------------------------------- K <= 128: A-stationary panel GEMM
// The factorisation's trailing updates and the sweep's lazy updates are rank-128 updates of
// a large fp32 matrix: K is one or two slabs, the output is what moves.  One CTA takes one
// 128-row block of A, keeps all of its planes in shared memory, and walks a run of n-tiles:
//   warp 0 : TMA, A once, then the B tiles of successive n-tiles through a 2-stage ring
//   warp 1 : tcgen05.mma into two alternating 128-column TMEM accumulators
//   warps 2..5 : epilogue of tile i (TMEM -> registers -> C += ...) while tile i+1 is multiplied
// so the read-modify-write of C, the B loads and the tensor pipe overlap.
constexpr int PANEL_MAX_RUN = 16;


__global__ void __launch_bounds__(GEMM_THREADS, 1) umma_panel_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                  const __grid_constant__ CUtensorMap map_b,
                                                                  const __grid_constant__ CUtensorMap map_c,
                                                                  const UmmaParams p, const int run) {
  const int m0 = blockIdx.y * TILE_M;
  const int n_tiles = (p.N + TILE_N - 1) / TILE_N;
  const int first = p.upper_tiles_only ? (int)blockIdx.y : 0;
  const int nt_begin = first + (int)blockIdx.x * run;
  int nt_end = nt_begin + run;
  if (nt_end > n_tiles) nt_end = n_tiles;
  if (nt_begin >= nt_end || m0 >= p.M) return;
  const int n_slabs = (p.K + SLAB_K - 1) / SLAB_K;  // 1 or 2
  const int count = nt_end - nt_begin;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_bytes = (uint32_t)(n_slabs * p.planes) * PLANE_TILE_BYTES;
  const uint32_t b_stage_bytes = (uint32_t)p.planes * PLANE_TILE_BYTES;
  const uint32_t b_base = smem_base + 2u * (uint32_t)p.planes * PLANE_TILE_BYTES;  // A always reserves two slabs
  __shared__ __align__(8) uint64_t bars[9];
  __shared__ uint32_t tmem_slot;
  const uint32_t a_full = smem_u32(&bars[0]);
  const uint32_t b_full = smem_u32(&bars[1]), b_empty = smem_u32(&bars[3]);
  const uint32_t acc_full = smem_u32(&bars[5]), acc_empty = smem_u32(&bars[7]);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int planes = p.planes;
  const uint32_t idesc = p.idesc;
  if (threadIdx.x == 0) {
    mbar_init(a_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(b_full + 8 * s, 1);
      mbar_init(b_empty + 8 * s, 1);
      mbar_init(acc_full + 8 * s, 1);
      mbar_init(acc_empty + 8 * s, 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // two alternating tiles, each with a leading and (more than one plane) a correction accumulator
  const uint32_t small_off = p.planes > 1 ? (uint32_t)TILE_N : 0u;
  const uint32_t acc_stride = p.planes > 1 ? 2u * TILE_N : (uint32_t)TILE_N;
  const uint32_t tmem_cols = 2u * acc_stride;
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = tmem_slot;
  // barriers and tensor memory are set up; from here on global memory is touched
  chain_wait();
  chain_release();

  // Producer and MMA warps run their loops with all 32 lanes (every lane waits on the
  // barriers); one lane issues the TMA / tcgen05 instructions.
  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(a_full, a_bytes);
      for (int s = 0; s < n_slabs; ++s)
        for (int pl = 0; pl < planes; ++pl)
          tma_load_3d(smem_base + (uint32_t)(s * planes + pl) * PLANE_TILE_BYTES, &map_a, a_full, s * SLAB_K + p.a_k0,
                      m0 + p.a_row0, pl);
    }
    int it = 0;
    bool ok = true;
    for (int i = 0; i < count && ok; ++i) {
      const int b_row = (nt_begin + i) * TILE_N;
      for (int s = 0; s < n_slabs; ++s, ++it) {
        const int st = it & 1;
        if (it >= 2 && !mbar_wait(b_empty + 8 * st, ((it >> 1) - 1) & 1, 11)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(b_full + 8 * st, b_stage_bytes);
          for (int pl = 0; pl < planes; ++pl)
            tma_load_3d(b_base + (uint32_t)st * b_stage_bytes + (uint32_t)pl * PLANE_TILE_BYTES, &map_b, b_full + 8 * st,
                        s * SLAB_K + p.b_k0, b_row + p.b_row0, pl);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    bool ok = mbar_wait(a_full, 0, 12);
    int it = 0;
    for (int i = 0; i < count && ok; ++i) {
      const int acc = i & 1;
      if (i >= 2) ok = mbar_wait(acc_empty + 8 * acc, ((i >> 1) - 1) & 1, 13);
      if (!ok) break;
      tc_fence_after();
      uint32_t accumulate = 0, accumulate_small = 0;
      for (int s = 0; s < n_slabs && ok; ++s, ++it) {
        const int st = it & 1;
        ok = mbar_wait(b_full + 8 * st, (it >> 1) & 1, 14);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_tile = smem_base + (uint32_t)(s * planes) * PLANE_TILE_BYTES;
          const uint32_t b_tile = b_base + (uint32_t)st * b_stage_bytes;
          issue_slab_any(planes, tmem_acc + (uint32_t)acc * acc_stride, small_off, a_tile, b_tile, idesc, accumulate, accumulate_small);
          umma_commit(b_empty + 8 * st);  // the stage is free once these MMAs have read it
        }
        __syncwarp();
      }
      if (ok && lane == 0) {
        umma_commit(acc_full + 8 * acc);
      }
      __syncwarp();
    }
  } else {
    const int q = warp & 3;
    const int row = m0 + q * 32 + lane;
    float* __restrict__ C = p.C;
    const bool vec_ok = (p.ldc & 3) == 0 && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
    // per-warp staging tile behind the operand buffers
    float* stage = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)) + 4u * (uint32_t)p.planes * PLANE_TILE_BYTES) +
                   (warp - 2) * 32 * STAGE_LD;
    bool ok = true;
    if (p.c_tma) {
      // Each warp owns two 4 KB boxes (32 rows x 128 B, 128-byte swizzle: no bank conflicts
      // when every lane writes its own row).  Box b is rewritten only after the bulk
      // operation issued from it two chunks earlier has read it.
      const uint32_t box0 = smem_base + 4u * (uint32_t)planes * PLANE_TILE_BYTES + (uint32_t)(warp - 2) * 8192u;
      const uint32_t my_row = box0 + (uint32_t)lane * 128u;
      const int y = m0 + q * 32;
      int chunk = 0;
      for (int i = 0; i < count && ok; ++i) {
        const int acc = i & 1;
        const int n0 = (nt_begin + i) * TILE_N;
        ok = mbar_wait(acc_full + 8 * acc, (i >> 1) & 1, 15);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < TILE_N / 32; ++c, ++chunk) {
          float v[32];
          tmem_ld32_sum(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * acc_stride + (uint32_t)(c * 32), small_off, v);
          if (c == TILE_N / 32 - 1) {
            // the accumulator is in registers: hand its TMEM columns back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + 8 * acc);
          }
          if (lane == 0) bulk_wait_read_1();
          __syncwarp();
          const uint32_t dst = my_row + (uint32_t)(chunk & 1) * 4096u;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst + (uint32_t)((j ^ (lane & 7)) << 4)),
                         "f"(p.alpha * v[4 * j]), "f"(p.alpha * v[4 * j + 1]), "f"(p.alpha * v[4 * j + 2]),
                         "f"(p.alpha * v[4 * j + 3])
                         : "memory");
          fence_async_smem();
          __syncwarp();
          const int x = n0 + c * 32;
          if (lane == 0 && y < p.M && x < p.N) {
            if (p.c_tma == 2) tma_add_2d(&map_c, box0 + (uint32_t)(chunk & 1) * 4096u, x, y);
            else tma_store_2d(&map_c, box0 + (uint32_t)(chunk & 1) * 4096u, x, y);
          }
          if (lane == 0) bulk_commit();
        }
      }
      if (lane == 0) bulk_wait_read_all();  // the boxes have left shared memory; the writes land before the grid completes
      __syncwarp();
    } else
    for (int i = 0; i < count && ok; ++i) {
      const int acc = i & 1;
      const int n0 = (nt_begin + i) * TILE_N;
      float* dst_row = C + (int64_t)row * p.ldc + n0;
      // tcgen05.ld is a warp-wide instruction: the choice of path must be uniform in the warp
      const bool whole = vec_ok && m0 + q * 32 + 32 <= p.M && n0 + TILE_N <= p.N;
      if (whole) {
        // Global accesses of the warp are whole 128-byte row segments: lane l works on row
        // 4*it + l/8, columns 4*(l%8).. of each 32-column chunk.  The accumulator arrives with
        // one row per lane, so it is turned through a 32 x 32 staging tile in shared memory.
        // All of C is requested before the accumulator is waited for: its latency overlaps the MMAs.
        float* cq = C + (int64_t)(m0 + q * 32 + (lane >> 3)) * p.ldc + n0 + (lane & 7) * 4;
        float4 old[TILE_N / 4];
        if (p.beta != 0.0f) {
#pragma unroll
          for (int c = 0; c < TILE_N / 32; ++c)
#pragma unroll
            for (int it = 0; it < 8; ++it)
              old[c * 8 + it] = *reinterpret_cast<const float4*>(cq + (int64_t)(4 * it) * p.ldc + c * 32);
        }
        ok = mbar_wait(acc_full + 8 * acc, (i >> 1) & 1, 15);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < TILE_N / 32; ++c) {
          float v[32];
          tmem_ld32_sum(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * acc_stride + (uint32_t)(c * 32), small_off, v);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(&stage[lane * STAGE_LD + 4 * j]) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const float4 a4 = *reinterpret_cast<const float4*>(&stage[(4 * it + (lane >> 3)) * STAGE_LD + (lane & 7) * 4]);
            float4 o = make_float4(p.alpha * a4.x, p.alpha * a4.y, p.alpha * a4.z, p.alpha * a4.w);
            if (p.beta != 0.0f) {
              const float4 od = old[c * 8 + it];
              o.x = fmaf(p.beta, od.x, o.x); o.y = fmaf(p.beta, od.y, o.y);
              o.z = fmaf(p.beta, od.z, o.z); o.w = fmaf(p.beta, od.w, o.w);
            }
            *reinterpret_cast<float4*>(cq + (int64_t)(4 * it) * p.ldc + c * 32) = o;
          }
          __syncwarp();
        }
      } else {
        ok = mbar_wait(acc_full + 8 * acc, (i >> 1) & 1, 15);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < TILE_N / 32; ++c) {
          const int col0 = n0 + c * 32;
          float v[32];
          tmem_ld32_sum(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * acc_stride + (uint32_t)(c * 32), small_off, v);
          if (row < p.M && col0 < p.N) {
            float* dst = dst_row + c * 32;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col0 + j < p.N) {
                float o = p.alpha * v[j];
                if (p.beta != 0.0f) o = fmaf(p.beta, dst[j], o);
                dst[j] = o;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + 8 * acc);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, tmem_cols);
  }
}

// ---------------------------------------------------------------- K > 128 with several planes: persistent streaming GEMM
// The far updates of the two-level factorisation and sweep: 512 of k at a time on a large fp32
// matrix, three planes per operand.  One CTA per SM walks the list of kept output tiles (tile
// number blockIdx.x + i * gridDim.x).  Both operands stream through a ring of two stages, each
// one 64-wide slab of k of A and of B (all planes: 96 KB with three), which keeps running across
// tiles; the accumulators alternate between two TMEM tiles, and the epilogue of tile i (C through
// the TMA unit where that is possible) runs under the MMAs of tile i + 1.  With one tile per CTA
// the tensor pipe idled through every prologue and epilogue (a quarter of a 512-deep tile).
//
// drain_slabs > 0 (with the TMA add only): the accumulator is handed to the epilogue after every
// drain_slabs slabs of k and added to C there, so the partial sums of K meet in round-to-nearest
// fp32 adds exactly as if the update had been issued as separate rank-128 updates.  The tensor
// core's own accumulation truncates; over 512 of k that bias is four times the one of 128, which
// the factorisation of an ill-conditioned Hessian does not forgive.  The adds of one tile still
// hit the L2 only: the tile is fetched from and written back to HBM once.
struct TileWalk {
  int m, n;
  __device__ __forceinline__ void seek(int idx, int n_tiles, int upper) {
    if (!upper) { m = idx / n_tiles; n = idx - m * n_tiles; return; }
    m = 0;
    for (;;) {                       // row m of the triangle keeps n_tiles - m tiles
      const int cnt = n_tiles - m;
      if (idx < cnt) { n = m + idx; return; }
      idx -= cnt;
      ++m;
    }
  }
};

// Unit u of a CTA's work: one accumulator's worth, `per_drain` slabs of k of one tile; the units
// of a tile follow one another.  (Letting two tiles take turns, so that the wait for the previous
// adds to a tile has a unit of slack, measured slower.)
struct UnitWalk {
  int tile, s0;
  __device__ __forceinline__ void seek(int u, int n_drains, int per_drain) {
    tile = u / n_drains;
    s0 = (u - tile * n_drains) * per_drain;
  }
};

__global__ void __launch_bounds__(GEMM_THREADS, 1) umma_stream_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                   const __grid_constant__ CUtensorMap map_b,
                                                                   const __grid_constant__ CUtensorMap map_c,
                                                                   const UmmaParams p, const int total) {
  const int n_tiles = (p.N + TILE_N - 1) / TILE_N;
  const int my_tiles = ((int)blockIdx.x < total) ? (total - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  if (my_tiles == 0) return;
  const int n_slabs = (p.K + SLAB_K - 1) / SLAB_K;
  const int per_drain = (p.drain_slabs > 0 && p.drain_slabs < n_slabs) ? p.drain_slabs : n_slabs;
  const int n_drains = (n_slabs + per_drain - 1) / per_drain;
  const int n_units = my_tiles * n_drains;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int planes = p.planes;
  const uint32_t stage_bytes = 2u * (uint32_t)planes * PLANE_TILE_BYTES;
  __shared__ __align__(8) uint64_t bars[8];
  __shared__ uint32_t tmem_slot;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[2]);
  const uint32_t acc_full = smem_u32(&bars[4]), acc_empty = smem_u32(&bars[6]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t idesc = p.idesc;
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
      mbar_init(acc_full + 8 * s, 1);
      mbar_init(acc_empty + 8 * s, 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const uint32_t small_off = planes > 1 ? (uint32_t)TILE_N : 0u;
  const uint32_t acc_stride = planes > 1 ? 2u * TILE_N : (uint32_t)TILE_N;
  const uint32_t tmem_cols = 2u * acc_stride;
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = tmem_slot;
  chain_wait();
  chain_release();

  if (warp == 0) {
    int it = 0;
    bool ok = true;
    for (int u = 0; u < n_units && ok; ++u) {
      UnitWalk uw;
      uw.seek(u, n_drains, per_drain);
      TileWalk w;
      w.seek((int)blockIdx.x + uw.tile * (int)gridDim.x, n_tiles, p.upper_tiles_only);
      const int a_row = w.m * TILE_M + p.a_row0, b_row = w.n * TILE_N + p.b_row0;
      const int s1 = (uw.s0 + per_drain) < n_slabs ? (uw.s0 + per_drain) : n_slabs;
      for (int s = uw.s0; s < s1; ++s, ++it) {
        const int st = it & 1;
        if (it >= 2 && !mbar_wait(empty0 + 8 * st, ((it >> 1) - 1) & 1, 41)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(full0 + 8 * st, stage_bytes);
          const uint32_t dst = smem_base + (uint32_t)st * stage_bytes;
          for (int pl = 0; pl < planes; ++pl) {
            tma_load_3d(dst + (uint32_t)pl * PLANE_TILE_BYTES, &map_a, full0 + 8 * st, s * SLAB_K + p.a_k0, a_row, pl);
            tma_load_3d(dst + (uint32_t)(planes + pl) * PLANE_TILE_BYTES, &map_b, full0 + 8 * st, s * SLAB_K + p.b_k0, b_row, pl);
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    int it = 0;
    bool ok = true;
    for (int u = 0; u < n_units && ok; ++u) {   // one accumulator handed to the epilogue per unit
      UnitWalk uw;
      uw.seek(u, n_drains, per_drain);
      const int acc = u & 1;
      if (u >= 2) ok = mbar_wait(acc_empty + 8 * acc, ((u >> 1) - 1) & 1, 42);
      if (!ok) break;
      tc_fence_after();
      uint32_t accumulate = 0, accumulate_small = 0;
      const int s1 = (uw.s0 + per_drain) < n_slabs ? (uw.s0 + per_drain) : n_slabs;
      for (int s = uw.s0; s < s1 && ok; ++s, ++it) {
        const int st = it & 1;
        ok = mbar_wait(full0 + 8 * st, (it >> 1) & 1, 43);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t a_tile = smem_base + (uint32_t)st * stage_bytes;
          const uint32_t b_tile = a_tile + (uint32_t)planes * PLANE_TILE_BYTES;
          issue_slab_any(planes, tmem_acc + (uint32_t)acc * acc_stride, small_off, a_tile, b_tile, idesc, accumulate, accumulate_small);
          umma_commit(empty0 + 8 * st);  // the stage is free once these MMAs have read it
        }
        __syncwarp();
      }
      if (ok && lane == 0) umma_commit(acc_full + 8 * acc);
      __syncwarp();
    }
  } else {
    const int q = warp & 3;
    bool ok = true;
    if (p.c_tma) {
      // Each warp owns two 4 KB boxes (32 rows x 128 B, 128-byte swizzle) behind the operand ring.
      const uint32_t box0 = smem_base + 2u * stage_bytes + (uint32_t)(warp - 2) * 8192u;
      const uint32_t my_row = box0 + (uint32_t)lane * 128u;
      int chunk = 0;
      for (int u = 0; u < n_units && ok; ++u) {
        UnitWalk uw;
        uw.seek(u, n_drains, per_drain);
        TileWalk w;
        w.seek((int)blockIdx.x + uw.tile * (int)gridDim.x, n_tiles, p.upper_tiles_only);
        const int n0 = w.n * TILE_N;
        const int y = w.m * TILE_M + q * 32;
        const int acc = u & 1;
        ok = mbar_wait(acc_full + 8 * acc, (u >> 1) & 1, 44);
        if (!ok) break;
        tc_fence_after();
        if (uw.s0 > 0) {
          // the adds of the previous part of this tile are done before this part's are issued:
          // every element receives its partial sums in the order of k, run after run
          if (lane == 0) bulk_wait_all();
          __syncwarp();
        }
#pragma unroll 1
        for (int c = 0; c < TILE_N / 32; ++c, ++chunk) {
          float v[32];
          tmem_ld32_sum(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * acc_stride + (uint32_t)(c * 32), small_off, v);
          if (c == TILE_N / 32 - 1) {
            // the accumulator is in registers: hand its TMEM columns back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + 8 * acc);
          }
          if (lane == 0) bulk_wait_read_1();
          __syncwarp();
          const uint32_t dst = my_row + (uint32_t)(chunk & 1) * 4096u;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst + (uint32_t)((j ^ (lane & 7)) << 4)),
                         "f"(p.alpha * v[4 * j]), "f"(p.alpha * v[4 * j + 1]), "f"(p.alpha * v[4 * j + 2]),
                         "f"(p.alpha * v[4 * j + 3])
                         : "memory");
          fence_async_smem();
          __syncwarp();
          const int x = n0 + c * 32;
          if (lane == 0 && y < p.M && x < p.N) {
            if (p.c_tma == 2) tma_add_2d(&map_c, box0 + (uint32_t)(chunk & 1) * 4096u, x, y);
            else tma_store_2d(&map_c, box0 + (uint32_t)(chunk & 1) * 4096u, x, y);
          }
          if (lane == 0) bulk_commit();
        }
      }
      if (lane == 0) bulk_wait_read_all();  // the boxes have left shared memory; the writes land before the grid completes
      __syncwarp();
    } else {
      float* stage_base = reinterpret_cast<float*>(smem_raw + (smem_base - smem_u32(smem_raw)) + 2u * stage_bytes);
      for (int i = 0; i < my_tiles && ok; ++i) {
        const int acc = i & 1;
        TileWalk w;
        w.seek((int)blockIdx.x + i * (int)gridDim.x, n_tiles, p.upper_tiles_only);
        ok = epilogue_tile<TILE_N>(p.alpha, p.beta, p.ldc, p.M, 0, p.C, w.m * TILE_M, w.n * TILE_N, p.N,
                                   tmem_acc + (uint32_t)acc * acc_stride, stage_base, warp, lane, n_slabs > 0, acc_full + 8 * acc,
                                   (uint32_t)((i >> 1) & 1), small_off);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty + 8 * acc);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, tmem_cols);
  }
}

// ---------------------------------------------------------------- operand planes
// dst plane pl, batch b, row r, k  <-  piece pl of src[b][r][k]; zero outside the logical
// (rows_b x K_b) extent up to the padded (rows_pad x K_pad) one.  32 x 32 tiles; when the
// source is contiguous along its row index the tile is transposed through shared memory
// so that both the global read and the global write are coalesced.
struct SplitParams {
  const void* src;
  int64_t rs, cs, bs;  // element strides of the source: row, k, batch
  int rows, K;         // logical extent per batch
  int rows_pad, K_pad;
  int planes;
  uint16_t* dst;
  int64_t plane_stride;
  // ragged last batch (see GemmDesc): rows_b = min(rows, row_total - b*row_step) etc.
  int row_total, row_step, k_total, k_step;
  // when set, 32 x 32 tiles whose k lies at or beyond the 128-block of their rows are skipped
  // (left unwritten): the caller only ever reads k-blocks in front of a row's own block
  int only_k_blocks_before_rows;
  // optional: every element of destination row r is divided by row_div[r] before it is split
  const float* row_div;
};

template <typename T>
__device__ __forceinline__ void split_store(float x, int planes, uint16_t* dst, int64_t idx, int64_t plane_stride);

template <>
__device__ __forceinline__ void split_store<__nv_bfloat16>(float x, int planes, uint16_t* dst, int64_t idx, int64_t ps) {
  __nv_bfloat16 h = __float2bfloat16_rn(x);
  dst[idx] = __bfloat16_as_ushort(h);
  if (planes > 1) {
    float r1 = x - __bfloat162float(h);
    __nv_bfloat16 m = __float2bfloat16_rn(r1);
    dst[idx + ps] = __bfloat16_as_ushort(m);
    if (planes > 2) {
      float r2 = r1 - __bfloat162float(m);
      dst[idx + 2 * ps] = __bfloat16_as_ushort(__float2bfloat16_rn(r2));
    }
  }
}
template <>
__device__ __forceinline__ void split_store<__half>(float x, int, uint16_t* dst, int64_t idx, int64_t) {
  dst[idx] = __half_as_ushort(__float2half_rn(x));  // fp16 activations enter as one exact plane
}

template <typename TIn, typename TPlane, bool TRANSPOSE>
__global__ void __launch_bounds__(256) split_planes_kernel(SplitParams p) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z;
  int rows = p.rows, K = p.K;
  if (p.row_step) { int left = p.row_total - b * p.row_step; rows = rows < left ? rows : left; }
  if (p.k_step) { int left = p.k_total - b * p.k_step; K = K < left ? K : left; }
  const TIn* __restrict__ src = static_cast<const TIn*>(p.src) + (int64_t)b * p.bs;
  const int r0 = blockIdx.y * 32, k0 = blockIdx.x * 32;
  if (p.only_k_blocks_before_rows && k0 >= (r0 / TILE_M) * TILE_M) return;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  if (TRANSPOSE) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int r = r0 + tx, k = k0 + ty + 8 * i;
      float x = (r < rows && k < K) ? to_float(src[(int64_t)r * p.rs + (int64_t)k * p.cs]) : 0.0f;
      if (p.row_div && r < rows) x = x / p.row_div[r];
      tile[ty + 8 * i][tx] = x;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rl = ty + 8 * i;
    const int r = r0 + rl, k = k0 + tx;
    if (r >= p.rows_pad || k >= p.K_pad) continue;
    float x;
    if (TRANSPOSE) x = tile[tx][rl];
    else {
      x = (r < rows && k < K) ? to_float(src[(int64_t)r * p.rs + (int64_t)k * p.cs]) : 0.0f;
      if (p.row_div && r < rows) x = x / p.row_div[r];
    }
    split_store<TPlane>(x, p.planes, p.dst, ((int64_t)b * p.rows_pad + r) * p.K_pad + k, p.plane_stride);
  }
}

// fp32 source whose row index is the contiguous one (a row-major matrix wanted transposed, the
// triangular factor for the sweep) -> up to three bf16 planes.  64 x 64 tiles: 256-byte rows on
// the global reads, 128-byte rows per plane on the writes, two k per thread.
__global__ void __launch_bounds__(256) split_transposed_f32_kernel(SplitParams p) {
  __shared__ float tile[64][65];  // tile[k][r]
  const int r0 = blockIdx.y * 64, k0 = blockIdx.x * 64;
  if (p.only_k_blocks_before_rows && k0 >= (r0 / TILE_M) * TILE_M) return;
  const float* __restrict__ src = static_cast<const float*>(p.src);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int k = k0 + warp + 8 * i;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = r0 + lane + 32 * h;
      tile[warp + 8 * i][lane + 32 * h] = (r < p.rows && k < p.K) ? __ldg(src + (int64_t)r * p.rs + (int64_t)k * p.cs) : 0.0f;
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rl = warp + 8 * i;
    const int r = r0 + rl, k = k0 + 2 * lane;
    if (r >= p.rows_pad || k >= p.K_pad) continue;  // K_pad is even
    float x0 = tile[2 * lane][rl], x1 = tile[2 * lane + 1][rl];
    if (p.row_div && r < p.rows) {
      const float d = __ldg(p.row_div + r);
      x0 = x0 / d;
      x1 = x1 / d;
    }
    uint16_t h0, m0, l0, h1, m1, l1;
    split_bf16x3(x0, h0, m0, l0);
    split_bf16x3(x1, h1, m1, l1);
    uint16_t* dst = p.dst + (int64_t)r * p.K_pad + k;
    *reinterpret_cast<uint32_t*>(dst) = (uint32_t)h0 | ((uint32_t)h1 << 16);
    if (p.planes > 1) *reinterpret_cast<uint32_t*>(dst + p.plane_stride) = (uint32_t)m0 | ((uint32_t)m1 << 16);
    if (p.planes > 2) *reinterpret_cast<uint32_t*>(dst + 2 * p.plane_stride) = (uint32_t)l0 | ((uint32_t)l1 << 16);
  }
}

// 16-bit activations whose row index is the contiguous one (X stored tokens x channels, wanted as
// channels x tokens): a plain transposing copy of one plane, 64 x 64 tiles, 128-byte rows on both
// the global reads and the global writes.  Zero outside (rows, K) up to (rows_pad, K_pad).
__global__ void __launch_bounds__(256) transpose16_kernel(const uint16_t* __restrict__ src, int64_t cs, int rows, int K,
                                                          int rows_pad, int K_pad, uint16_t* __restrict__ dst) {
  __shared__ uint16_t tile[64][66];  // tile[k][r]
  const int r0 = blockIdx.y * 64, k0 = blockIdx.x * 64;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool pair_ok = (cs & 1) == 0 && (reinterpret_cast<uintptr_t>(src) & 3) == 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int k = k0 + warp + 8 * i, r = r0 + 2 * lane;
    uint32_t v = 0;
    if (k < K) {
      const uint16_t* s = src + (int64_t)k * cs + r;
      if (pair_ok && r + 1 < rows) v = __ldg(reinterpret_cast<const uint32_t*>(s));
      else v = (r < rows ? (uint32_t)__ldg(s) : 0u) | (r + 1 < rows ? (uint32_t)__ldg(s + 1) << 16 : 0u);
    }
    *reinterpret_cast<uint32_t*>(&tile[warp + 8 * i][2 * lane]) = v;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + warp + 8 * i, k = k0 + 2 * lane;
    if (r >= rows_pad || k >= K_pad) continue;  // K_pad is even
    const uint32_t v = (uint32_t)tile[2 * lane][warp + 8 * i] | ((uint32_t)tile[2 * lane + 1][warp + 8 * i] << 16);
    *reinterpret_cast<uint32_t*>(dst + (int64_t)r * K_pad + k) = v;
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encoder(EncodeTiledFn* out) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    MQ_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres));
    MQ_REQUIRE(sym && qres == cudaDriverEntryPointSuccess, MQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  *out = fn;
  return MQ_OK;
}

int encode_map(const PlaneSet& ps, CUtensorMap* map) {
  EncodeTiledFn enc;
  MQ_TRY(get_encoder(&enc));
  cuuint64_t dims[3] = {(cuuint64_t)ps.K_pad, (cuuint64_t)ps.total_rows, (cuuint64_t)ps.planes};
  cuuint64_t strides[2] = {(cuuint64_t)ps.K_pad * 2, (cuuint64_t)ps.K_pad * 2 * (cuuint64_t)ps.total_rows};
  cuuint32_t box[3] = {SLAB_K, TILE_M, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, ps.fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ps.base, dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MQ_REQUIRE(r == CUDA_SUCCESS, MQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (K_pad=%d rows=%lld planes=%d)", (int)r,
             ps.K_pad, (long long)ps.total_rows, ps.planes);
  return MQ_OK;
}

// fp32 matrix C (M x N, row stride ldc) as a 2-D map with 32 x 32 boxes for the TMA epilogue.
int encode_c_map(float* C, int64_t ldc, int M, int N, CUtensorMap* map) {
  EncodeTiledFn enc;
  MQ_TRY(get_encoder(&enc));
  cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  cuuint64_t strides[1] = {(cuuint64_t)ldc * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, C, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MQ_REQUIRE(r == CUDA_SUCCESS, MQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d for C (M=%d N=%d ldc=%lld)", (int)r, M, N,
             (long long)ldc);
  return MQ_OK;
}

int pad_to(int x, int a) { return (x + a - 1) / a * a; }

template <typename TIn, typename TPlane>
int launch_split(const SplitParams& sp, int batch, cudaStream_t st) {
  dim3 grid((unsigned)(sp.K_pad / 32), (unsigned)(sp.rows_pad / 32), (unsigned)batch);
  ProfScope prof(PROF_SPLIT, (double)batch * sp.rows_pad * sp.K_pad * (sizeof(TIn) + 2.0 * sp.planes), 0.0, st);
  if (sp.rs == 1 && sp.cs != 1)
    split_planes_kernel<TIn, TPlane, true><<<grid, 256, 0, st>>>(sp);
  else
    split_planes_kernel<TIn, TPlane, false><<<grid, 256, 0, st>>>(sp);
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}

int make_planes(const void* src, int in_dtype, int64_t rs, int64_t cs, int64_t bs, int rows, int K, int batch, int planes,
                int row_total, int row_step, int k_total, int k_step, Workspace& ws, PlaneSet* out, cudaStream_t st,
                bool only_k_blocks_before_rows = false, const float* row_div = nullptr) {
  PlaneSet ps;
  ps.planes = in_dtype == MQ_F32 ? planes : 1;
  ps.rows_pad = pad_to(rows, TILE_M);
  ps.K_pad = pad_to(K, SLAB_K);
  ps.total_rows = (int64_t)batch * ps.rows_pad;
  ps.fp16 = in_dtype == MQ_F16;
  const size_t elems = (size_t)ps.planes * ps.total_rows * ps.K_pad;
  ps.base = ws.take<uint16_t>(elems);
  MQ_REQUIRE(ps.base, MQ_ERR_WORKSPACE, "tensor engine: workspace too small for %zu plane elements", elems);
  SplitParams sp;
  sp.src = src; sp.rs = rs; sp.cs = cs; sp.bs = bs;
  sp.rows = rows; sp.K = K; sp.rows_pad = ps.rows_pad; sp.K_pad = ps.K_pad;
  sp.planes = ps.planes; sp.dst = ps.base; sp.plane_stride = ps.total_rows * ps.K_pad;
  sp.row_total = row_total; sp.row_step = row_step; sp.k_total = k_total; sp.k_step = k_step;
  sp.only_k_blocks_before_rows = only_k_blocks_before_rows ? 1 : 0;
  sp.row_div = row_div;
  if (in_dtype != MQ_F32 && rs == 1 && cs != 1 && batch == 1 && !row_step && !k_step) {
    // bf16 / fp16 bit patterns pass through unchanged
    dim3 grid((unsigned)ceil_div(ps.K_pad, 64), (unsigned)ceil_div(ps.rows_pad, 64), 1);
    ProfScope prof(PROF_SPLIT, (double)ps.rows_pad * ps.K_pad * 4.0, 0.0, st);
    transpose16_kernel<<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(src), cs, rows, K, ps.rows_pad, ps.K_pad, ps.base);
    MQ_LAUNCH_CHECK();
    *out = ps;
    return MQ_OK;
  }
  if (in_dtype == MQ_F32 && rs == 1 && cs != 1 && batch == 1 && !row_step && !k_step) {
    dim3 grid((unsigned)ceil_div(ps.K_pad, 64), (unsigned)ceil_div(ps.rows_pad, 64), 1);
    ProfScope prof(PROF_SPLIT, (double)ps.rows_pad * ps.K_pad * (4.0 + 2.0 * ps.planes), 0.0, st);
    split_transposed_f32_kernel<<<grid, 256, 0, st>>>(sp);
    MQ_LAUNCH_CHECK();
    *out = ps;
    return MQ_OK;
  }
  switch (in_dtype) {
    case MQ_F32: MQ_TRY((launch_split<float, __nv_bfloat16>(sp, batch, st))); break;
    case MQ_BF16: MQ_TRY((launch_split<__nv_bfloat16, __nv_bfloat16>(sp, batch, st))); break;
    default: MQ_TRY((launch_split<__half, __half>(sp, batch, st)));
  }
  *out = ps;
  return MQ_OK;
}

int configure_once() {
  static bool done[64] = {};
  int dev = 0;
  MQ_CUDA(cudaGetDevice(&dev));
  if (!done[dev & 63]) {
    MQ_CUDA(cudaFuncSetAttribute(umma_gemm_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    MQ_CUDA(cudaFuncSetAttribute(umma_gemm_persistent_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024));
    MQ_CUDA(cudaFuncSetAttribute(umma_gemm_persistent_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024));
    MQ_CUDA(cudaFuncSetAttribute(umma_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    MQ_CUDA(cudaFuncSetAttribute(umma_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    done[dev & 63] = true;
  }
  return MQ_OK;
}

int launch_umma(const GemmDesc& d, const PlaneSet& A, const PlaneSet& B, cudaStream_t st) {
  MQ_TRY(configure_once());
  CUtensorMap map_a, map_b;
  MQ_TRY(encode_map(A, &map_a));
  MQ_TRY(encode_map(B, &map_b));
  UmmaParams p;
  p.C = d.C; p.ldc = d.ldc; p.c_bs = d.c_bs;
  p.M = d.M; p.N = d.N; p.K = d.K;
  p.alpha = d.alpha; p.beta = d.beta;
  p.upper_tiles_only = d.upper_tiles_only; p.a_upper = d.a_upper; p.b_upper = d.b_upper;
  p.n_total = d.n_total; p.n_step = d.n_step; p.k_follows_n = d.k_follows_n;
  p.mirror = d.mirror_to_lower;
  p.a_rows_pad = A.rows_pad; p.b_rows_pad = B.rows_pad;
  p.a_row0 = (int)A.row0; p.a_k0 = A.k0; p.b_row0 = (int)B.row0; p.b_k0 = B.k0;
  p.planes = A.planes;
  p.drain_slabs = 0;
  p.nterms = 0;
  for (int i = 0; i < A.planes; ++i)
    for (int j = 0; i + j < A.planes; ++j) ++p.nterms;
  const uint32_t fmt = A.fp16 ? 0u : 1u;  // operand format: 0 = fp16, 1 = bf16
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(TILE_N >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
  const int stage_bytes = A.planes * 2 * PLANE_TILE_BYTES;
  int stages = (192 * 1024) / stage_bytes;
  if (stages > 3) stages = 3;  // one-plane GEMMs: 97 KB per CTA, so two CTAs share an SM and overlap epilogue with MMA
  p.stages = stages;
  const size_t smem = (size_t)stages * stage_bytes + 1024;
  dim3 grid((unsigned)ceil_div(d.N, TILE_N), (unsigned)ceil_div(d.M, TILE_M), (unsigned)d.batch);
  double flop_alg = 0.0, flop_issued = 0.0;
  if (g_profile_on) gemm_work(d, SLAB_K, &flop_alg, &flop_issued, p.nterms);
  const bool panel_route = d.K <= 2 * SLAB_K && d.batch == 1 && !d.a_upper && !d.b_upper && !d.n_step && d.K > 0 && !d.mirror_to_lower;
  const bool deep_route = !panel_route && A.planes > 1 && d.batch == 1 && !d.a_upper && !d.b_upper && !d.n_step && !d.mirror_to_lower &&
                          d.K > 2 * SLAB_K;
  ProfScope prof(deep_route ? PROF_UMMA_DEEP : PROF_UMMA_GEMM, flop_alg, flop_issued, st);
  if (d.K <= 2 * SLAB_K && d.batch == 1 && !d.a_upper && !d.b_upper && !d.n_step && d.K > 0 && !d.mirror_to_lower) {
    // rank-<=128 update: keep A in shared memory and walk runs of n-tiles
    const int m_tiles = (int)ceil_div(d.M, TILE_M), n_tiles = (int)ceil_div(d.N, TILE_N);
    const long long tiles = d.upper_tiles_only ? (long long)n_tiles * (n_tiles + 1) / 2 : (long long)m_tiles * n_tiles;
    // Pick the run length that minimises (waves of CTAs) x (fixed cost of a CTA + run): long
    // runs pay the barrier/TMEM/first-load cost once, but the CTA count should fill the 148 SMs
    // without a nearly empty last wave.
    int run = 1;
    {
      double best = 1e30;
      for (int cand = 1; cand <= PANEL_MAX_RUN; ++cand) {
        long long ctas = 0;
        for (int m = 0; m < m_tiles; ++m) {
          const int cnt = d.upper_tiles_only ? n_tiles - m : n_tiles;
          if (cnt > 0) ctas += (cnt + cand - 1) / cand;
        }
        const double waves = (double)((ctas + 147) / 148);
        const double cost = waves * (4.0 + cand);
        if (cost < best) { best = cost; run = cand; }
      }
    }
    if (d.compact) run = n_tiles < PANEL_MAX_RUN ? n_tiles : PANEL_MAX_RUN;
    dim3 pgrid((unsigned)ceil_div(n_tiles, run), (unsigned)m_tiles, 1);
    // C goes through the TMA unit when the map can be built (16-byte aligned rows, and a beta
    // that a plain store (0) or an add at the L2 (1) expresses) and every SM has at least two
    // tiles: with fewer, the warps' own prefetched read-modify-write has the shorter latency.
    // N must be a multiple of 4: the unit clips a box at the tensor's edge in 16-byte units,
    // so a ragged last column would spill up to three elements past C's row.
    CUtensorMap map_c;
    memset(&map_c, 0, sizeof(map_c));
    p.c_tma = 0;
    if (tiles >= 2 * 148 && (d.ldc & 3) == 0 && (d.N & 3) == 0 && (reinterpret_cast<uintptr_t>(d.C) & 15) == 0 && (d.beta == 0.0f || d.beta == 1.0f)) {
      MQ_TRY(encode_c_map(d.C, d.ldc, d.M, d.N, &map_c));
      p.c_tma = d.beta == 0.0f ? 1 : 2;
    }
    const size_t staging = p.c_tma ? (size_t)4 * 2 * 4096 : (size_t)STAGE_BYTES;
    const size_t psmem = (size_t)4 * A.planes * PLANE_TILE_BYTES + 1024 + staging;  // A: two slabs, B: two stages, staging
    MQ_CUDA(launch_chained(true, umma_panel_kernel, pgrid, dim3(GEMM_THREADS), psmem, st, map_a, map_b, map_c, p, run));
  } else if (A.planes > 1 && d.batch == 1 && !d.a_upper && !d.b_upper && !d.n_step && !d.mirror_to_lower && d.K > 2 * SLAB_K) {
    // deep update with several planes: persistent streaming kernel
    const int m_tiles = (int)ceil_div(d.M, TILE_M), n_tiles = (int)ceil_div(d.N, TILE_N);
    long long tiles = (long long)m_tiles * n_tiles;
    if (d.upper_tiles_only) {
      const int rows = m_tiles < n_tiles ? m_tiles : n_tiles;   // row m keeps n_tiles - m tiles
      tiles = (long long)rows * n_tiles - (long long)rows * (rows - 1) / 2;
    }
    CUtensorMap map_c;
    memset(&map_c, 0, sizeof(map_c));
    p.c_tma = 0;
    if ((d.ldc & 3) == 0 && (d.N & 3) == 0 && (reinterpret_cast<uintptr_t>(d.C) & 15) == 0 && (d.beta == 0.0f || d.beta == 1.0f)) {
      MQ_TRY(encode_c_map(d.C, d.ldc, d.M, d.N, &map_c));
      p.c_tma = d.beta == 0.0f ? 1 : 2;
    }
    p.drain_slabs = (d.k_round > 0 && p.c_tma == 2) ? d.k_round / SLAB_K : 0;
    const size_t staging = p.c_tma ? (size_t)4 * 2 * 4096 : (size_t)STAGE_BYTES;
    const size_t ssmem = (size_t)4 * A.planes * PLANE_TILE_BYTES + 1024 + staging;   // two stages of A and B slabs, staging
    MQ_CUDA(launch_chained(true, umma_stream_kernel, dim3((unsigned)(tiles < 148 ? tiles : 148)), dim3(GEMM_THREADS), ssmem, st,
                           map_a, map_b, map_c, p, (int)tiles));
  } else {
    if (A.planes == 1 && d.batch == 1 && !d.a_upper && !d.b_upper && !d.n_step && d.N >= 256) {
      // one product per element: 128 x 256 tiles, four 48 KB stages, one persistent CTA per SM
      p.stages = PERSIST_STAGES;
      p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(PERSIST_TN >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
      const int my_tiles = (int)ceil_div(d.M, TILE_M), nx_tiles = (int)ceil_div(d.N, PERSIST_TN);
      long long n_work = 0;
      for (int ty = 0; ty < my_tiles; ++ty) {
        const int tx0 = d.upper_tiles_only ? (ty * TILE_M) / PERSIST_TN : 0;
        if (nx_tiles > tx0) n_work += nx_tiles - tx0;
      }
      const size_t wsmem = (size_t)PERSIST_STAGES * (PLANE_TILE_BYTES + PERSIST_TN * SLAB_K * 2) + STAGE_BYTES + 1024;
      umma_gemm_persistent_kernel<false><<<(unsigned)(n_work < 148 ? n_work : 148), GEMM_THREADS, wsmem, st>>>(map_a, map_b, p, (int)n_work);
    } else {
      umma_gemm_kernel<128><<<grid, GEMM_THREADS, smem, st>>>(map_a, map_b, p);
    }
  }
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}

}  // namespace

int gemm_tensor_planes(const GemmDesc& d, const PlaneSet& A, const PlaneSet& B, cudaStream_t st) {
  if (d.M <= 0 || d.N <= 0 || d.batch <= 0) return MQ_OK;
  MQ_REQUIRE(A.planes == B.planes && A.planes >= 1 && A.planes <= 3 && A.fp16 == B.fp16, MQ_ERR_ARGUMENT,
             "tensor engine: operand plane sets do not match");
  if (d.k_round > 0 && d.K > d.k_round) {
    MQ_REQUIRE(d.k_round % SLAB_K == 0 && d.beta == 1.0f && d.batch == 1, MQ_ERR_ARGUMENT,
               "tensor engine: k_round needs a multiple of %d, beta == 1 and one batch", SLAB_K);
    const bool c_tma = (d.ldc & 3) == 0 && (d.N & 3) == 0 && (reinterpret_cast<uintptr_t>(d.C) & 15) == 0;
    if (!c_tma || A.planes == 1) {
      // no add at the L2 for this C (or one plane, which the streaming kernel does not take):
      // the same partial sums as separate updates
      for (int k = 0; k < d.K; k += d.k_round) {
        GemmDesc part = d;
        part.K = (d.K - k) < d.k_round ? (d.K - k) : d.k_round;
        part.k_round = 0;
        PlaneSet a = A, b = B;
        a.k0 += k; b.k0 += k;
        MQ_TRY(launch_umma(part, a, b, st));
      }
      return MQ_OK;
    }
  }
  return launch_umma(d, A, B, st);
}

int make_planes_f32(const float* src, int64_t rs, int64_t cs, int rows, int K, int planes, uint16_t* dst, PlaneSet* out,
                    cudaStream_t st, bool only_k_blocks_before_rows, const float* row_div) {
  Workspace ws(dst, plane_set_bytes(rows, K, planes));
  return make_planes(src, MQ_F32, rs, cs, 0, rows, K, 1, planes, 0, 0, 0, 0, ws, out, st, only_k_blocks_before_rows, row_div);
}

size_t engine_workspace_bytes(int64_t M, int64_t N, int64_t K, int math, int split) {
  if (math != MQ_MATH_TENSOR) return 0;
  const size_t kp = (size_t)pad_to((int)K, SLAB_K);
  const size_t a = (size_t)split * (size_t)pad_to((int)M, TILE_M) * kp * 2;
  const size_t b = (size_t)split * (size_t)pad_to((int)N, TILE_N) * kp * 2;
  return align_up(a, 256) + align_up(b, 256);
}

int gemm_tensor_f32(const GemmDesc& d, int split, Workspace ws, cudaStream_t st) {
  if (d.M <= 0 || d.N <= 0 || d.batch <= 0) return MQ_OK;
  MQ_REQUIRE(split >= 1 && split <= 3, MQ_ERR_ARGUMENT, "tensor engine: split must be 1, 2 or 3 (got %d)", split);
  PlaneSet A, B;
  // A planes [m][k]: the k extent follows the ragged N when k_follows_n is set
  MQ_TRY(make_planes(d.A, MQ_F32, d.a_rs, d.a_cs, d.a_bs, d.M, d.K, d.batch, split, 0, 0,
                     d.k_follows_n ? d.n_total : 0, d.k_follows_n ? d.n_step : 0, ws, &A, st));
  const bool same = d.A == d.B && d.a_rs == d.b_cs && d.a_cs == d.b_rs && d.M == d.N && d.batch == 1 && !d.n_step;
  if (same) {
    B = A;  // symmetric rank-k update: B^T is A
  } else {
    // B planes [n][k] = B[k][n]
    MQ_TRY(make_planes(d.B, MQ_F32, d.b_cs, d.b_rs, d.b_bs, d.N, d.K, d.batch, split, d.n_step ? d.n_total : 0, d.n_step,
                       d.k_follows_n ? d.n_total : 0, d.k_follows_n ? d.n_step : 0, ws, &B, st));
  }
  return launch_umma(d, A, B, st);
}

size_t hessian_accum_tensor_workspace_bytes(int x_dtype, int64_t m, int64_t C, int split) {
  const size_t planes = x_dtype == MQ_F32 ? (size_t)split : 1;
  return align_up(planes * (size_t)pad_to((int)C, TILE_M) * (size_t)pad_to((int)(m > 0 ? m : 1), SLAB_K) * 2, 256);
}

int hessian_accum_tensor(const void* X, int x_dtype, int64_t m, int64_t C, int64_t ldx, float* H, int64_t ldh, float beta,
                         float alpha, int split, Workspace& ws, cudaStream_t st) {
  MQ_REQUIRE(split >= 1 && split <= 3, MQ_ERR_ARGUMENT, "mq_hessian_accum: split must be 1, 2 or 3 (got %d)", split);
  if (x_dtype != MQ_F32 && m > 0 && C >= PERSIST_TN && (ldx & 7) == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0) {
    // 16-bit activations are read where they lie: no transposed copy, no workspace
    MQ_TRY(configure_once());
    EncodeTiledFn enc;
    MQ_TRY(get_encoder(&enc));
    CUtensorMap map_x;
    cuuint64_t dims[2] = {(cuuint64_t)C, (cuuint64_t)m};
    cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
    cuuint32_t box[2] = {64, 64};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&map_x, x_dtype == MQ_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                     const_cast<void*>(X), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MQ_REQUIRE(r == CUDA_SUCCESS, MQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d for X (tokens=%lld C=%lld ldx=%lld)",
               (int)r, (long long)m, (long long)C, (long long)ldx);
    UmmaParams p = {};
    p.C = H; p.ldc = ldh;
    p.M = (int)C; p.N = (int)C; p.K = (int)m;
    p.alpha = alpha; p.beta = beta;
    p.upper_tiles_only = 1; p.mirror = 1;
    p.planes = 1; p.nterms = 1; p.stages = PERSIST_STAGES;
    const uint32_t fmt = x_dtype == MQ_F16 ? 0u : 1u;
    // both operands MN-major (bits 15 and 16)
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(PERSIST_TN >> 3) << 17) |
              ((uint32_t)(TILE_M >> 4) << 24);
    const int my_tiles = (int)ceil_div(C, TILE_M), nx_tiles = (int)ceil_div(C, PERSIST_TN);
    long long n_work = 0;
    for (int ty = 0; ty < my_tiles; ++ty) {
      const int tx0 = (ty * TILE_M) / PERSIST_TN;
      if (nx_tiles > tx0) n_work += nx_tiles - tx0;
    }
    const size_t wsmem = (size_t)PERSIST_STAGES * (PLANE_TILE_BYTES + PERSIST_TN * SLAB_K * 2) + STAGE_BYTES + 1024;
    ProfScope prof(PROF_UMMA_GEMM, (double)m * C * (C + 1), 2.0 * (double)n_work * TILE_M * PERSIST_TN * pad_to((int)m, SLAB_K), st);
    umma_gemm_persistent_kernel<true><<<(unsigned)(n_work < 148 ? n_work : 148), GEMM_THREADS, wsmem, st>>>(map_x, map_x, p,
                                                                                                          (int)n_work);
    MQ_LAUNCH_CHECK();
    return MQ_OK;
  }
  GemmDesc g;
  g.C = H; g.ldc = ldh;
  g.M = (int)C; g.N = (int)C; g.K = (int)m;
  g.alpha = alpha; g.beta = beta;
  g.upper_tiles_only = 1;
  PlaneSet A;
  if (m > 0) {
    // planes of X^T: row = channel, k = token
    MQ_TRY(make_planes(X, x_dtype, 1, ldx, 0, (int)C, (int)m, 1, split, 0, 0, 0, 0, ws, &A, st));
  } else {
    // nothing to add: only the beta scaling remains, done by the epilogue on an empty K range
    A.planes = 1; A.rows_pad = pad_to((int)C, TILE_M); A.K_pad = SLAB_K; A.total_rows = A.rows_pad;
    A.base = ws.take<uint16_t>((size_t)A.rows_pad * SLAB_K);
    MQ_REQUIRE(A.base, MQ_ERR_WORKSPACE, "mq_hessian_accum: workspace too small");
  }
  g.mirror_to_lower = 1;  // the epilogue stores every block above the diagonal transposed as well
  return launch_umma(g, A, A, st);
}

}  // namespace mq

extern "C" int mq_engine_fault(int* host_out) {
  using namespace mq;
  MQ_REQUIRE(host_out, MQ_ERR_ARGUMENT, "mq_engine_fault: null pointer");
  MQ_CUDA(cudaMemcpyFromSymbol(host_out, g_engine_fault, sizeof(int)));
  return MQ_OK;
}

extern "C" int mq_engine_fault_clear(void) {
  using namespace mq;
  const int zero = 0;
  MQ_CUDA(cudaDeviceSynchronize());
  MQ_CUDA(cudaMemcpyToSymbol(g_engine_fault, &zero, sizeof(int)));
  return MQ_OK;
}
