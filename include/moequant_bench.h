/*
 * moequant_bench.h - measurement hooks of libmoequant_sm100.so.
 *
 * Not part of the product ABI (moequant.h): nothing on the quantization path calls these, and a
 * binding of the library for the reference project does not need them.  They exist so that a
 * benchmark can count the library's own launches and time its kernel families without a profiler.
 */
#ifndef MOEQUANT_BENCH_H_
#define MOEQUANT_BENCH_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Number of CUDA kernels this library has launched in this process (host-side counter). */
long long mq_launch_count(void);

/* Per-kernel timing for benchmarks: between mq_profile_begin() and mq_profile_end() every
 * launch of the kernel families below is bracketed by CUDA events on its own stream.
 * mq_profile_end synchronises the device and fills four arrays of MQ_PROFILE_KINDS entries:
 * launches, summed milliseconds, and two work figures (GEMM kinds: algorithmic flop and
 * issued tensor flop; sweep: algorithmic bytes and flop; split/pack: bytes).
 * Not thread-safe; meant for one benchmarking thread.  */
#define MQ_PROFILE_KINDS 9
enum { MQ_PROF_UMMA_GEMM = 0, MQ_PROF_SIMT_GEMM = 1, MQ_PROF_SWEEP_TILE = 2, MQ_PROF_CHOL_DIAG = 3,
       MQ_PROF_TRSM = 4, MQ_PROF_SPLIT = 5, MQ_PROF_PACK = 6, MQ_PROF_OTHER = 7,
       MQ_PROF_UMMA_DEEP = 8 /* tensor GEMMs with more than 128 of k and several planes: the streaming kernel */ };
int mq_profile_begin(void);
int mq_profile_end(int64_t* launches, double* milliseconds, double* work, double* work2);

#ifdef __cplusplus
}
#endif
#endif /* MOEQUANT_BENCH_H_ */
