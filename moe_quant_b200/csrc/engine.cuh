// Picks the arithmetic for a dense contraction: fp32 CUDA cores or tcgen05
// tensor cores on split-bf16 planes.  One Engine lives for the duration of one
// C-ABI call and carves its scratch out of that call's workspace.
#pragma once

#include "gemm.cuh"

namespace mq {

// Scratch the tensor-core path needs for a GEMM whose operands are at most
// (M x K) and (K x N) fp32: the bf16 planes of both operands.
size_t engine_workspace_bytes(int64_t M, int64_t N, int64_t K, int math, int split);

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
