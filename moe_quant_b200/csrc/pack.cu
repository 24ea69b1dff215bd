// int4 -> int32 packing in the compressed-tensors layout, and the matching
// dequantizer.  Both are pure bandwidth kernels: every byte of the code matrix is
// read once with 16-byte loads, every output byte written once.
//
// Replaces pack_weight -> compressed_tensors.pack_to_int32
// (pack_quantized_model.py:57-75) and dequantize_linear_weight
// (src/quant_utils.py:243-256).
#include "common.cuh"
#include "profile.cuh"

namespace mq {

constexpr int kPackThreads = 256;

__device__ __forceinline__ uint32_t pack8(uint32_t lo4, uint32_t hi4) {
  // lo4 holds codes c0..c3 as bytes (c0 lowest), hi4 holds c4..c7.  With every code
  // < 16 the sum of shifted codes equals the OR of the nibbles.
  uint32_t w = (lo4 & 0xFu) | ((lo4 >> 4) & 0xF0u) | ((lo4 >> 8) & 0xF00u) | ((lo4 >> 12) & 0xF000u);
  uint32_t v = (hi4 & 0xFu) | ((hi4 >> 4) & 0xF0u) | ((hi4 >> 8) & 0xF00u) | ((hi4 >> 12) & 0xF000u);
  return w | (v << 16);
}

// Fast path: symmetric (zero == 8, nibble == code), C % 16 == 0, 16-byte aligned base.
// One thread turns 16 codes into two words, four such vectors per trip with all four loads
// issued before the first is used: a 22 MB matrix is one short wave of CTAs, so what counts is
// how many bytes every thread has in flight, not how many trips it makes.
constexpr int kPackUnroll = 4;
__global__ void __launch_bounds__(kPackThreads) pack_int4_vec16(const uint4* __restrict__ codes,
                                                                uint2* __restrict__ packed, int64_t n_vec) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < n_vec; i0 += stride * kPackUnroll) {
    uint4 c[kPackUnroll];
#pragma unroll
    for (int u = 0; u < kPackUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      c[u] = i < n_vec ? __ldcs(codes + i) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < kPackUnroll; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < n_vec) __stcs(packed + i, make_uint2(pack8(c[u].x, c[u].y), pack8(c[u].z, c[u].w)));
    }
  }
}

// General path: any C, optional per-group int8 zero points.  One thread per word.
// Follows the library arithmetic literally: u = uint8(int8(code) - zero + 8), the
// word is the wrapping int32 sum of u << 4i, columns past C contribute 0.
__global__ void __launch_bounds__(kPackThreads) pack_int4_general(const uint8_t* __restrict__ codes, int64_t R,
                                                                  int64_t C, const int8_t* __restrict__ zero,
                                                                  int64_t group, int32_t* __restrict__ packed) {
  int64_t words_per_row = (C + 7) / 8;
  int64_t n = R * words_per_row;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t n_groups = zero ? C / group : 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t r = i / words_per_row;
    int64_t k = i - r * words_per_row;
    uint32_t w = 0;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      int64_t c = k * 8 + t;
      if (c < C) {
        int8_t v = (int8_t)codes[r * C + c];
        int8_t z = zero ? zero[r * n_groups + c / group] : (int8_t)8;
        uint8_t u = (uint8_t)(int8_t)(v - z + 8);
        w += (uint32_t)u << (4 * t);
      }
    }
    packed[i] = (int32_t)w;
  }
}

template <int DT>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ codes, int64_t R, int64_t C,
                                                         const float* __restrict__ scale,
                                                         const float* __restrict__ zero_pts, int64_t group, float zero,
                                                         typename StorageOf<DT>::type* __restrict__ out) {
  using T = typename StorageOf<DT>::type;
  int64_t n = R * C;
  int64_t G = C / group;
  int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    // C % 4 == 0 is checked on the host, so four consecutive elements share a row.
    int64_t r = i / C;
    int64_t c = i - r * C;
    uint32_t q4 = *reinterpret_cast<const uint32_t*>(codes + i);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      int64_t gi = r * G + (c + t) / group;
      float s = __ldg(scale + gi);
      float z = zero_pts ? __ldg(zero_pts + gi) : zero;
      float q = (float)((q4 >> (8 * t)) & 0xFFu);
      out[i + t] = from_float<T>((q - z) * s);
    }
  }
}

static int grid_for(int64_t work_items, int threads) {
  int64_t blocks = ceil_div(work_items, threads);
  int64_t cap = 148 * 8;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace mq

extern "C" int mq_pack_int4(const uint8_t* codes, int64_t R, int64_t C, const int8_t* zero_i8, int64_t group,
                            int32_t* packed, void* stream) {
  using namespace mq;
  MQ_REQUIRE(R >= 0 && C >= 0, MQ_ERR_ARGUMENT, "mq_pack_int4: negative shape R=%lld C=%lld", (long long)R, (long long)C);
  if (R == 0 || C == 0) return MQ_OK;
  MQ_REQUIRE(codes && packed, MQ_ERR_ARGUMENT, "mq_pack_int4: null pointer");
  MQ_REQUIRE(aligned(packed, 4), MQ_ERR_ALIGNMENT, "mq_pack_int4: packed must be 4-byte aligned");
  if (zero_i8) {
    MQ_REQUIRE(group > 0 && C % group == 0, MQ_ERR_ARGUMENT, "mq_pack_int4: group %lld does not divide C=%lld",
               (long long)group, (long long)C);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ProfScope prof(PROF_PACK, 1.5 * (double)R * (double)C, 0.0, st);
  if (!zero_i8 && C % 16 == 0 && aligned(codes, 16) && aligned(packed, 8)) {
    int64_t n_vec = R * C / 16;
    pack_int4_vec16<<<grid_for(ceil_div(n_vec, kPackUnroll), kPackThreads), kPackThreads, 0, st>>>(
        reinterpret_cast<const uint4*>(codes), reinterpret_cast<uint2*>(packed), n_vec);
  } else {
    int64_t n = R * ((C + 7) / 8);
    pack_int4_general<<<grid_for(n, kPackThreads), kPackThreads, 0, st>>>(codes, R, C, zero_i8, group, packed);
  }
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}

extern "C" int mq_dequantize(const uint8_t* codes, int64_t R, int64_t C, const float* scale, const float* zero_pts,
                             int64_t group, int bits, int out_dtype, void* out, void* stream) {
  using namespace mq;
  MQ_REQUIRE(R >= 0 && C >= 0, MQ_ERR_ARGUMENT, "mq_dequantize: negative shape");
  if (R == 0 || C == 0) return MQ_OK;
  MQ_REQUIRE(codes && scale && out, MQ_ERR_ARGUMENT, "mq_dequantize: null pointer");
  MQ_REQUIRE(bits >= 2 && bits <= 8, MQ_ERR_ARGUMENT, "mq_dequantize: bits=%d", bits);
  MQ_REQUIRE(valid_dtype(out_dtype), MQ_ERR_ARGUMENT, "mq_dequantize: bad dtype %d", out_dtype);
  MQ_REQUIRE(group > 0 && C % group == 0, MQ_ERR_ARGUMENT, "mq_dequantize: group %lld does not divide C=%lld",
             (long long)group, (long long)C);
  MQ_REQUIRE(C % 4 == 0 && aligned(codes, 4), MQ_ERR_UNSUPPORTED, "mq_dequantize: needs C %% 4 == 0 and 4-byte aligned codes");
  float zero = 0.5f * (float)(1 << bits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int grid = grid_for(R * C / 4, 256);
  switch (out_dtype) {
    case MQ_F32:
      dequantize_kernel<MQ_F32><<<grid, 256, 0, st>>>(codes, R, C, scale, zero_pts, group, zero, static_cast<float*>(out));
      break;
    case MQ_BF16:
      dequantize_kernel<MQ_BF16><<<grid, 256, 0, st>>>(codes, R, C, scale, zero_pts, group, zero, static_cast<__nv_bfloat16*>(out));
      break;
    default:
      dequantize_kernel<MQ_F16><<<grid, 256, 0, st>>>(codes, R, C, scale, zero_pts, group, zero, static_cast<__half*>(out));
  }
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}
