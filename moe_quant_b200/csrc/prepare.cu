// Hessian preparation (NaN guard, dead channels, zero-column masking, damping)
// and the symmetric absmax grid.  All of it is one or two passes over H / W, i.e.
// HBM-bound, and everything stays on the device: no host round trip for the
// `.any().item()` of the reference (src/gptq.py:141).
#include "common.cuh"

namespace mq {

// ---------------------------------------------------------------- NaN guard
__global__ void __launch_bounds__(256) nan_scan_kernel(const float* __restrict__ H, int64_t C, int64_t ldh,
                                                       mq_layer_flags* flags) {
  // C % 4 == 0 and ldh % 4 == 0 (checked on the host): rows are float4-addressable.  A thread
  // keeps its column and walks rows, four independent loads per step, no index division.
  const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  bool bad = false;
  if (c < C) {
    const float* col = H + c;
    int64_t r = blockIdx.y;
    for (; r + 3 * (int64_t)gridDim.y < C; r += 4 * (int64_t)gridDim.y) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldg(reinterpret_cast<const float4*>(col + (r + u * (int64_t)gridDim.y) * ldh));
#pragma unroll
      for (int u = 0; u < 4; ++u) bad |= (v[u].x != v[u].x) | (v[u].y != v[u].y) | (v[u].z != v[u].z) | (v[u].w != v[u].w);
    }
    for (; r < C; r += gridDim.y) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(col + r * ldh));
      bad |= (v.x != v.x) | (v.y != v.y) | (v.z != v.z) | (v.w != v.w);
    }
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicExch(&flags->nan_hessian, 1);
}

__global__ void __launch_bounds__(256) identity_if_nan_kernel(float* __restrict__ H, int64_t C, int64_t ldh,
                                                              const mq_layer_flags* flags) {
  if (flags->nan_hessian == 0) return;
  int64_t n = C * C;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int64_t r = i / C, c = i - r * C;
    H[r * ldh + c] = (r == c) ? 1.0f : 0.0f;
  }
}

// ---------------------------------------------------------------- column masks
// nonzero[c] = 1 when any W[r, c] != 0.  Threads of a warp read consecutive columns.
__global__ void __launch_bounds__(256) column_nonzero_kernel(const float* __restrict__ W, int64_t R, int64_t C,
                                                             int64_t ldw, int rows_per_block,
                                                             int* __restrict__ nonzero) {
  int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  int64_t r0 = (int64_t)blockIdx.y * rows_per_block;
  int64_t r1 = r0 + rows_per_block < R ? r0 + rows_per_block : R;
  bool nz = false;
  for (int64_t r = r0; r < r1; ++r) nz |= (__ldg(W + r * ldw + c) != 0.0f);
  if (nz) nonzero[c] = 1;
}

// One block: lists the masked channels (diag(H)==0, or an all-zero weight column).
// list[0] = count, list[1..] = channel indices (order is irrelevant).
__global__ void __launch_bounds__(1024) build_mask_kernel(const float* __restrict__ H, int64_t C, int64_t ldh,
                                                          const int* __restrict__ nonzero, int* __restrict__ list,
                                                          mq_layer_flags* flags) {
  __shared__ int n_masked, n_dead, n_zero;
  if (threadIdx.x == 0) n_masked = n_dead = n_zero = 0;
  __syncthreads();
  for (int64_t c = threadIdx.x; c < C; c += blockDim.x) {
    bool dead = H[c * ldh + c] == 0.0f;
    // The reference zeroes W[:, dead] before looking for all-zero columns, so a dead
    // channel is always also a zero column (src/gptq.py:145-152, 224).
    bool zero_col = dead || (nonzero != nullptr && nonzero[c] == 0);
    if (dead) atomicAdd(&n_dead, 1);
    if (zero_col) {
      atomicAdd(&n_zero, 1);
      int slot = atomicAdd(&n_masked, 1);
      list[1 + slot] = (int)c;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    list[0] = n_masked;
    flags->dead_channels = n_dead;
    flags->zero_columns = n_zero;
  }
}

// Rows and columns of the masked channels become those of the identity; their weight
// column becomes zero.
__global__ void __launch_bounds__(256) apply_mask_kernel(float* __restrict__ H, int64_t C, int64_t ldh,
                                                         float* __restrict__ W, int64_t R, int64_t ldw,
                                                         const int* __restrict__ list) {
  int n_masked = list[0];
  if (n_masked == 0) return;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (int k = 0; k < n_masked; ++k) {
    int64_t c = list[1 + k];
    for (int64_t i = tid; i < C; i += stride) {
      float v = (i == c) ? 1.0f : 0.0f;
      H[c * ldh + i] = v;
      H[i * ldh + c] = v;
    }
    if (W != nullptr) {
      for (int64_t r = tid; r < R; r += stride) W[r * ldw + c] = 0.0f;
    }
  }
}

// One block: H[i,i] += rel_damp * mean(diag H).
__global__ void __launch_bounds__(1024) damp_kernel(float* __restrict__ H, int64_t C, int64_t ldh, float rel_damp) {
  __shared__ float partial[32];
  __shared__ float damp_s;
  float acc = 0.0f;
  for (int64_t c = threadIdx.x; c < C; c += blockDim.x) acc += H[c * ldh + c];
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.0f;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) damp_s = rel_damp * (v / (float)C);
  }
  __syncthreads();
  float damp = damp_s;
  for (int64_t c = threadIdx.x; c < C; c += blockDim.x) H[c * ldh + c] += damp;
}

// ---------------------------------------------------------------- absmax grid
// One warp walks one (row, group) segment at a time with float4 loads.
template <int DT>
__global__ void __launch_bounds__(256) absmax_scales_kernel(const float* __restrict__ W, int64_t R, int64_t C,
                                                            int64_t ldw, int64_t group, float two_over_maxq,
                                                            float* __restrict__ scale) {
  int64_t G = C / group;
  int64_t n_seg = R * G;
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t seg = warp; seg < n_seg; seg += n_warps) {
    int64_t r = seg / G, gi = seg - r * G;
    const float* p = W + r * ldw + gi * group;
    float m = 0.0f;
    if ((group & 3) == 0) {
      for (int64_t k = lane * 4; k < group; k += 128) {
        float4 v = __ldg(reinterpret_cast<const float4*>(p + k));
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
      }
    } else {
      for (int64_t k = lane; k < group; k += 32) m = fmaxf(m, fabsf(__ldg(p + k)));
    }
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) {
      // (2/maxq) * absmax, then + 1e-12, each rounded to fp32, then through the layer dtype:
      // the operation order of src/quant_utils.py:95-96.
      float s = __fadd_rn(__fmul_rn(two_over_maxq, m), 1e-12f);
      scale[seg] = round_through<DT>(s);
    }
  }
}

// ---------------------------------------------------------------- MSE scale search
// One warp per (row, group): the absmax scale s0 is shrunk by each candidate factor p_i,
//   s_i = round_to_dtype(s0 * p_i),  loss_i = sum_c |dequant(quant(x_c; s_i)) - x_c|^norm,
// and replaced by s0 * p_argmin rounded through the dtype (mse_scale_triton_kernel,
// src/quant_utils.py:104-139).  |d|^norm is exp(norm * log|d|) as in tl_pow (src/quant_utils.py:25-27),
// which is 0 for d == 0.  Of equal losses the first candidate wins; candidates with equal losses
// almost always have equal rounded scales, so the choice among them does not change the result.
template <int DT>
__global__ void __launch_bounds__(256) mse_scales_kernel(const float* __restrict__ W, int64_t R, int64_t C, int64_t ldw,
                                                         int64_t group, float maxq, float zero,
                                                         const float* __restrict__ p, int p_size, float norm,
                                                         float* __restrict__ scale) {
  const int64_t G = C / group;
  const int64_t n_seg = R * G;
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t seg = warp; seg < n_seg; seg += n_warps) {
    const int64_t r = seg / G, gi = seg - r * G;
    const float* x = W + r * ldw + gi * group;
    const float s0 = scale[seg];
    float best = 0.0f;
    int best_i = -1;
    for (int i = 0; i < p_size; ++i) {
      const float s = round_through<DT>(__fmul_rn(s0, __ldg(p + i)));
      float loss = 0.0f;
      for (int64_t k = lane; k < group; k += 32) {
        const float xv = __ldg(x + k);
        const float q = fminf(fmaxf(floorf(__fadd_rn(__fadd_rn(__fdiv_rn(xv, s), zero), 0.5f)), 0.0f), maxq);
        const float y = round_through<DT>(__fmul_rn(q - zero, s));
        loss += __expf(__logf(fabsf(y - xv)) * norm);
      }
      for (int o = 16; o > 0; o >>= 1) loss += __shfl_xor_sync(0xffffffffu, loss, o);
      if (best_i < 0 || loss < best) { best = loss; best_i = i; }
    }
    if (lane == 0 && best_i >= 0) scale[seg] = round_through<DT>(__fmul_rn(s0, __ldg(p + best_i)));
  }
}

// ---------------------------------------------------------------- fp32 working copy
template <typename T>
__global__ void __launch_bounds__(256) to_fp32_kernel(const T* __restrict__ src, float* __restrict__ dst, int64_t n) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = to_float(src[i]);
}

int launch_to_fp32(const void* src, int dtype, float* dst, int64_t n, cudaStream_t st) {
  if (n == 0) return MQ_OK;
  int grid = (int)(ceil_div(n, 256) < 148 * 8 ? ceil_div(n, 256) : 148 * 8);
  switch (dtype) {
    case MQ_F32:
      MQ_CUDA(cudaMemcpyAsync(dst, src, n * sizeof(float), cudaMemcpyDeviceToDevice, st));
      return MQ_OK;
    case MQ_BF16:
      to_fp32_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(src), dst, n);
      break;
    case MQ_F16:
      to_fp32_kernel<<<grid, 256, 0, st>>>(static_cast<const __half*>(src), dst, n);
      break;
    default:
      set_error("bad dtype %d", dtype);
      return MQ_ERR_ARGUMENT;
  }
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}

}  // namespace mq

extern "C" size_t mq_hessian_prepare_workspace_bytes(int64_t C) {
  if (C < 0) return 0;
  // nonzero[C] + list[1 + C], each rounded up to 256 bytes
  return mq::align_up((size_t)C * sizeof(int), 256) + mq::align_up((size_t)(C + 1) * sizeof(int), 256);
}

extern "C" int mq_hessian_prepare(float* H, int64_t C, int64_t ldh, float* W, int64_t R, int64_t ldw, float rel_damp,
                                  mq_layer_flags* flags, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace mq;
  MQ_REQUIRE(H && flags, MQ_ERR_ARGUMENT, "mq_hessian_prepare: null H or flags");
  MQ_REQUIRE(C > 0 && ldh >= C, MQ_ERR_ARGUMENT, "mq_hessian_prepare: bad C=%lld ldh=%lld", (long long)C, (long long)ldh);
  MQ_REQUIRE(C % 4 == 0 && ldh % 4 == 0 && aligned(H, 16), MQ_ERR_ALIGNMENT,
             "mq_hessian_prepare: needs C %% 4 == 0, ldh %% 4 == 0 and a 16-byte aligned H");
  if (W) MQ_REQUIRE(R > 0 && ldw >= C, MQ_ERR_ARGUMENT, "mq_hessian_prepare: bad R=%lld ldw=%lld", (long long)R, (long long)ldw);
  Workspace ws(workspace, workspace_bytes);
  int* nonzero = ws.take<int>(C);
  int* list = ws.take<int>(C + 1);
  MQ_REQUIRE(nonzero && list, MQ_ERR_WORKSPACE, "mq_hessian_prepare: workspace of %zu bytes is too small", workspace_bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  MQ_CUDA(cudaMemsetAsync(flags, 0, sizeof(mq_layer_flags), st));
  {
    const unsigned gx = (unsigned)ceil_div(C / 4, 256);
    unsigned gy = (unsigned)(148 * 8 / gx);
    if (gy < 1) gy = 1;
    if ((int64_t)gy > C) gy = (unsigned)C;
    nan_scan_kernel<<<dim3(gx, gy), 256, 0, st>>>(H, C, ldh, flags);
  }
  MQ_LAUNCH_CHECK();
  identity_if_nan_kernel<<<148 * 4, 256, 0, st>>>(H, C, ldh, flags);
  MQ_LAUNCH_CHECK();
  if (W) {
    MQ_CUDA(cudaMemsetAsync(nonzero, 0, C * sizeof(int), st));
    const int rows_per_block = 64;
    dim3 grid((unsigned)ceil_div(C, 256), (unsigned)ceil_div(R, rows_per_block));
    column_nonzero_kernel<<<grid, 256, 0, st>>>(W, R, C, ldw, rows_per_block, nonzero);
    MQ_LAUNCH_CHECK();
  }
  build_mask_kernel<<<1, 1024, 0, st>>>(H, C, ldh, W ? nonzero : nullptr, list, flags);
  MQ_LAUNCH_CHECK();
  apply_mask_kernel<<<148, 256, 0, st>>>(H, C, ldh, W, R, ldw, list);
  MQ_LAUNCH_CHECK();
  damp_kernel<<<1, 1024, 0, st>>>(H, C, ldh, rel_damp);
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}

extern "C" int mq_absmax_scales(const float* W, int64_t R, int64_t C, int64_t ldw, int64_t group, int bits,
                                int out_dtype, float* scale, void* stream) {
  using namespace mq;
  MQ_REQUIRE(W && scale, MQ_ERR_ARGUMENT, "mq_absmax_scales: null pointer");
  MQ_REQUIRE(R > 0 && C > 0 && ldw >= C, MQ_ERR_ARGUMENT, "mq_absmax_scales: bad shape R=%lld C=%lld ldw=%lld",
             (long long)R, (long long)C, (long long)ldw);
  MQ_REQUIRE(group > 0 && C % group == 0, MQ_ERR_ARGUMENT, "mq_absmax_scales: group %lld does not divide C=%lld",
             (long long)group, (long long)C);
  MQ_REQUIRE(bits >= 2 && bits <= 8, MQ_ERR_ARGUMENT, "mq_absmax_scales: bits=%d", bits);
  MQ_REQUIRE(valid_dtype(out_dtype), MQ_ERR_ARGUMENT, "mq_absmax_scales: bad dtype %d", out_dtype);
  if (group % 4 == 0) {
    MQ_REQUIRE(aligned(W, 16) && ldw % 4 == 0, MQ_ERR_ALIGNMENT, "mq_absmax_scales: W must be 16-byte aligned with ldw %% 4 == 0");
  }
  float two_over_maxq = 2.0f / (float)((1 << bits) - 1);
  int64_t n_seg = R * (C / group);
  int grid = (int)(ceil_div(n_seg, 8) < 148 * 8 ? ceil_div(n_seg, 8) : 148 * 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (out_dtype) {
    case MQ_F32:
      absmax_scales_kernel<MQ_F32><<<grid, 256, 0, st>>>(W, R, C, ldw, group, two_over_maxq, scale);
      break;
    case MQ_BF16:
      absmax_scales_kernel<MQ_BF16><<<grid, 256, 0, st>>>(W, R, C, ldw, group, two_over_maxq, scale);
      break;
    default:
      absmax_scales_kernel<MQ_F16><<<grid, 256, 0, st>>>(W, R, C, ldw, group, two_over_maxq, scale);
  }
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}

extern "C" int mq_mse_scales(const float* W, int64_t R, int64_t C, int64_t ldw, int64_t group, int bits, int out_dtype,
                             const float* shrink, int n_shrink, float norm, float* scale, void* stream) {
  using namespace mq;
  MQ_REQUIRE(W && scale && shrink, MQ_ERR_ARGUMENT, "mq_mse_scales: null pointer");
  MQ_REQUIRE(R > 0 && C > 0 && ldw >= C && n_shrink > 0, MQ_ERR_ARGUMENT, "mq_mse_scales: bad shape R=%lld C=%lld ldw=%lld n=%d",
             (long long)R, (long long)C, (long long)ldw, n_shrink);
  MQ_REQUIRE(group > 0 && C % group == 0, MQ_ERR_ARGUMENT, "mq_mse_scales: group %lld does not divide C=%lld",
             (long long)group, (long long)C);
  MQ_REQUIRE(bits >= 2 && bits <= 8, MQ_ERR_ARGUMENT, "mq_mse_scales: bits=%d", bits);
  MQ_REQUIRE(valid_dtype(out_dtype), MQ_ERR_ARGUMENT, "mq_mse_scales: bad dtype %d", out_dtype);
  const float maxq = (float)((1 << bits) - 1), zero = 0.5f * (float)(1 << bits);
  const int64_t n_seg = R * (C / group);
  const int grid = (int)(ceil_div(n_seg, 8) < 148 * 8 ? ceil_div(n_seg, 8) : 148 * 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (out_dtype) {
    case MQ_F32:
      mse_scales_kernel<MQ_F32><<<grid, 256, 0, st>>>(W, R, C, ldw, group, maxq, zero, shrink, n_shrink, norm, scale);
      break;
    case MQ_BF16:
      mse_scales_kernel<MQ_BF16><<<grid, 256, 0, st>>>(W, R, C, ldw, group, maxq, zero, shrink, n_shrink, norm, scale);
      break;
    default:
      mse_scales_kernel<MQ_F16><<<grid, 256, 0, st>>>(W, R, C, ldw, group, maxq, zero, shrink, n_shrink, norm, scale);
  }
  MQ_LAUNCH_CHECK();
  return MQ_OK;
}

// ---------------------------------------------------------------------------- no-allocation variant
// Some hosts of this library have no way to hand over scratch memory: a plain C program that
// was given nothing but the H and W pointers by another runtime, a plug-in running inside a
// process whose allocator it must not call (all device memory already belongs to a pool it
// does not control), or code on a path where cudaMalloc's implicit device synchronisation is
// not acceptable.  For them the channel lists of the preparation step live in this
// file-scope array instead of a caller workspace.  It is sized for kNoAllocMaxChannels
// input channels (about 256 KB) and every GPU that loads the library carries it until the
// process exits.
namespace mq {
constexpr int64_t kNoAllocMaxChannels = 32768;
constexpr size_t kNoAllocScratchBytes = ((kNoAllocMaxChannels * 4 + 255) / 256) * 256 + (((kNoAllocMaxChannels + 1) * 4 + 255) / 256) * 256;
static __device__ __align__(256) unsigned char g_prepare_scratch[kNoAllocScratchBytes];
}  // namespace mq

extern "C" int mq_hessian_prepare_noalloc(float* H, int64_t C, int64_t ldh, float* W, int64_t R, int64_t ldw,
                                          float rel_damp, mq_layer_flags* flags, void* stream) {
  using namespace mq;
  MQ_REQUIRE(C > 0, MQ_ERR_ARGUMENT, "mq_hessian_prepare_noalloc: bad C=%lld", (long long)C);
  MQ_REQUIRE(C <= kNoAllocMaxChannels, MQ_ERR_UNSUPPORTED,
             "mq_hessian_prepare_noalloc: C=%lld is beyond the built-in scratch (%lld channels); "
             "use mq_hessian_prepare with a caller-provided workspace",
             (long long)C, (long long)kNoAllocMaxChannels);
  MQ_REQUIRE(mq_hessian_prepare_workspace_bytes(C) <= kNoAllocScratchBytes, MQ_ERR_UNSUPPORTED,
             "mq_hessian_prepare_noalloc: built-in scratch too small for C=%lld", (long long)C);
  // In host code the array's name is only a handle; the kernels need its device address,
  // which differs per GPU.  Looked up once per device, with that device current.
  static void* device_address[64] = {};
  int dev = -1;
  MQ_CUDA(cudaGetDevice(&dev));
  MQ_REQUIRE(dev >= 0 && dev < 64, MQ_ERR_UNSUPPORTED, "mq_hessian_prepare_noalloc: device ordinal %d not supported", dev);
  if (device_address[dev] == nullptr) {
    void* p = nullptr;
    MQ_CUDA(cudaGetSymbolAddress(&p, g_prepare_scratch));
    MQ_REQUIRE(p != nullptr, MQ_ERR_CUDA, "mq_hessian_prepare_noalloc: no device address for the built-in scratch");
    device_address[dev] = p;
  }
  // Same kernels, same order as mq_hessian_prepare; the zero-initialised parts of the scratch
  // (column flags, list length) are cleared by that sequence on every call.
  return mq_hessian_prepare(H, C, ldh, W, R, ldw, rel_damp, flags, device_address[dev], kNoAllocScratchBytes, stream);
}
