// Shared by the sweep's kernels: the argument block of a tile launch.
#pragma once

#include <utility>

#include "engine.cuh"

namespace mq {

constexpr int SWEEP_TILE = 128;

// eight codes below 16, held as bytes in two words (lowest byte = first column) -> one word of nibbles
__device__ __forceinline__ uint32_t pack_nibbles(uint32_t lo4, uint32_t hi4) {
  const uint32_t w = (lo4 & 0xFu) | ((lo4 >> 4) & 0xF0u) | ((lo4 >> 8) & 0xF00u) | ((lo4 >> 12) & 0xF000u);
  const uint32_t v = (hi4 & 0xFu) | ((hi4 >> 4) & 0xF0u) | ((hi4 >> 8) & 0xF00u) | ((hi4 >> 12) & 0xF000u);
  return w | (v << 16);
}

struct SweepArgs {
  const float* W; int64_t ldw; int R;
  const float* U; int64_t ldu;
  const float* scale; const float* zero; int64_t group, s_rs, s_gs;
  float maxq, zero_default;
  uint8_t* codes; int64_t C;
  int32_t* packed;   // optional (R, C/8) int32: the same codes, eight 4-bit nibbles per word
  void* deq; float* err;
  int i1, nb;
  const float* Worig; int64_t ldwo;
  uint16_t* err_planes; int64_t plane_stride; int n_planes;
  int err_ld;   // row stride of err / err_planes (both already point at this tile's k window)
  int bits;
};


}  // namespace mq
