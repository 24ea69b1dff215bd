// Shared helpers of the sm_100a GPTQ engine: status handling, dtype rounding,
// launch checks.  Everything here is internal to the shared library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <utility>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/moequant.h"

namespace mq {

void set_error(const char* fmt, ...);

#define MQ_REQUIRE(cond, code, ...)  \
  do {                               \
    if (!(cond)) {                   \
      mq::set_error(__VA_ARGS__);    \
      return (code);                 \
    }                                \
  } while (0)

#define MQ_CUDA(expr)                                                              \
  do {                                                                             \
    cudaError_t _e = (expr);                                                       \
    if (_e != cudaSuccess) {                                                       \
      mq::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return MQ_ERR_CUDA;                                                          \
    }                                                                              \
  } while (0)

extern long long g_launches;  // kernels launched by this library in this process
#define MQ_LAUNCH_CHECK()         \
  do {                            \
    ++mq::g_launches;             \
    MQ_CUDA(cudaGetLastError());  \
  } while (0)

// ---------------------------------------------------------------- programmatic dependent launch
// The kernels of the layer loop (diagonal block, panel solve, rank-128 update, sweep tile) are
// a chain of small dependent launches.  Launched through launch_chained, a kernel may be
// made resident while its predecessor in the stream still runs; it must call
// chain_wait() before it touches global memory (that returns once every earlier grid has
// completed and its writes are visible) and then chain_release(), which lets its own successor
// be made resident.  Releasing only after the wait keeps at most one waiting grid on the GPU.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(bool chained, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained ? 1 : 0;  // not chained: an ordinary launch, fully ordered after its predecessor
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

#define MQ_TRY(expr)              \
  do {                            \
    int _s = (expr);              \
    if (_s != MQ_OK) return _s;   \
  } while (0)

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Bump allocator over the caller's workspace; every carve-out is 256-byte aligned.
struct Workspace {
  char* base;
  size_t size;
  size_t used;
  Workspace(void* p, size_t n) : base(static_cast<char*>(p)), size(n), used(0) {}
  template <typename T>
  T* take(size_t count) {
    size_t bytes = align_up(count * sizeof(T), 256);
    if (base == nullptr || used + bytes > size) return nullptr;
    T* r = reinterpret_cast<T*>(base + used);
    used += bytes;
    return r;
  }
};

// Round an fp32 value through the layer dtype with round-to-nearest-even, the
// "round_fp" of the reference (src/quant_utils.py:37-39, 57-58).
template <int DT>
__device__ __forceinline__ float round_through(float x) {
  if constexpr (DT == MQ_BF16) {
    return __bfloat162float(__float2bfloat16_rn(x));
  } else if constexpr (DT == MQ_F16) {
    return __half2float(__float2half_rn(x));
  } else {
    return x;
  }
}

template <int DT>
struct StorageOf;
template <>
struct StorageOf<MQ_F32> { using type = float; };
template <>
struct StorageOf<MQ_BF16> { using type = __nv_bfloat16; };
template <>
struct StorageOf<MQ_F16> { using type = __half; };

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ float from_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }

inline size_t dtype_size(int dt) { return dt == MQ_F32 ? 4 : 2; }
inline bool valid_dtype(int dt) { return dt == MQ_F32 || dt == MQ_BF16 || dt == MQ_F16; }

}  // namespace mq
