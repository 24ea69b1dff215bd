// Optional per-kernel timing: CUDA events recorded on the launching stream around
// each launch of the kernel families below, switched on by mq_profile_begin().
// Off by default; when off the hooks cost one predictable branch.
#pragma once

#include "common.cuh"

namespace mq {

enum ProfKind { PROF_UMMA_GEMM = 0, PROF_SIMT_GEMM = 1, PROF_SWEEP_TILE = 2, PROF_CHOL_DIAG = 3, PROF_TRSM = 4,
                PROF_SPLIT = 5, PROF_PACK = 6, PROF_OTHER = 7, PROF_UMMA_DEEP = 8, PROF_KINDS = 9 };

extern bool g_profile_on;
void prof_open(int kind, double work, double work2, cudaStream_t st);
void prof_close(cudaStream_t st);

// RAII bracket around one kernel launch.  `work` and `work2` are two work figures of the
// launch (e.g. algorithmic flop and issued tensor flop, or algorithmic bytes).
struct ProfScope {
  cudaStream_t st;
  bool on;
  ProfScope(int kind, double work, double work2, cudaStream_t s) : st(s), on(g_profile_on) {
    if (on) prof_open(kind, work, work2, st);
  }
  ~ProfScope() {
    if (on) prof_close(st);
  }
};

}  // namespace mq
