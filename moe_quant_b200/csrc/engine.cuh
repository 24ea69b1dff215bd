// Picks the arithmetic for a dense contraction: fp32 CUDA cores or tcgen05
// tensor cores on split-bf16 planes.  One Engine lives for the duration of one
// C-ABI call and carves its scratch out of that call's workspace.
#pragma once

#include "gemm.cuh"

namespace mq {

// Scratch the tensor-core path needs for a GEMM whose operands are at most
// (M x K) and (K x N) fp32: the bf16 planes of both operands.
size_t engine_workspace_bytes(int64_t M, int64_t N, int64_t K, int math, int split);

// 16-bit planes of one GEMM operand, K-major: element (plane, row, k) at
// base[(plane * total_rows + row) * K_pad + k].  rows are padded to 128, k to 64, so that every
// TMA box is fully inside the buffer.  row0 / k0 shift the origin: the operand of a GEMM may be a
// window of a larger plane buffer (e.g. one 128-wide k range of the planes of the whole factor).
struct PlaneSet {
  uint16_t* base = nullptr;
  int planes = 0;
  int64_t total_rows = 0;  // batch * rows_pad
  int rows_pad = 0;        // rows one batch occupies
  int K_pad = 0;
  bool fp16 = false;
  int64_t row0 = 0;
  int k0 = 0;
};

inline int64_t pad_rows(int64_t rows) { return (rows + 127) / 128 * 128; }
inline int64_t pad_k(int64_t k) { return (k + 63) / 64 * 64; }
inline size_t plane_set_bytes(int64_t rows, int64_t K, int planes) {
  return align_up((size_t)planes * (size_t)pad_rows(rows) * (size_t)pad_k(K) * 2, 256);
}

// x -> hi + mid + lo with bf16 pieces; each residual is exact in fp32.
__device__ __forceinline__ void split_bf16x3(float x, uint16_t& hi, uint16_t& mid, uint16_t& lo) {
  const __nv_bfloat16 h = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(h);
  const __nv_bfloat16 m = __float2bfloat16_rn(r1);
  const float r2 = r1 - __bfloat162float(m);
  hi = __bfloat16_as_ushort(h);
  mid = __bfloat16_as_ushort(m);
  lo = __bfloat16_as_ushort(__float2bfloat16_rn(r2));
}

// Tensor-core GEMM whose operands are already planes (d.A / d.B and their strides are ignored;
// d.K is the reduction length starting at k0 of each set).  Both sets must have the same
// number of planes.
int gemm_tensor_planes(const GemmDesc& d, const PlaneSet& A, const PlaneSet& B, cudaStream_t st);

// fp32 matrix (rows x K, element (r,k) at src[r*rs + k*cs]) -> planes, zero padded.
// only_k_blocks_before_rows: write only the part with k in a 128-block in front of the row's own
// 128-block (the strictly upper blocks of a triangular factor stored transposed); the rest of
// the buffer stays unwritten and must not be read.  row_div (optional, device): destination row r is
// divided by row_div[r] before the split.
int make_planes_f32(const float* src, int64_t rs, int64_t cs, int rows, int K, int planes, uint16_t* dst, PlaneSet* out,
                    cudaStream_t st, bool only_k_blocks_before_rows = false, const float* row_div = nullptr);

// Tensor-core GEMM on fp32 operands that are split into `split` bf16 planes on the fly.
int gemm_tensor_f32(const GemmDesc& d, int split, Workspace ws, cudaStream_t st);

struct Engine {
  int math;
  int split;
  Workspace ws;  // private view of what is left of the call's workspace
  cudaStream_t st;
  Engine(int math_, int split_, const Workspace& remaining, cudaStream_t st_)
      : math(math_), split(split_), ws(remaining.base ? remaining.base + remaining.used : nullptr,
                                        remaining.base ? remaining.size - remaining.used : 0), st(st_) {}
  int gemm(const GemmDesc& d) {
    if (math == MQ_MATH_TENSOR) return gemm_tensor_f32(d, split, ws, st);
    return gemm_simt(d, MQ_F32, st);
  }
};

}  // namespace mq
