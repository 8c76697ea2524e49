// Quantize / Dequantize at the boundary between the float and the uint8 part of a network.
//
// Reference behaviour: QuantizeUtil<float, uint8_t> (mace/core/quantize.h:128-215) as the
// Quantize and Dequantize operators call it (mace/ops/quantize.cc:31-115):
//   quantize:    q = Saturate<uint8_t>(roundf(zero_point + (1 / scale) * x))
//   find range:  min x, max x (FindMinMax, quantize.h:90-102), then AdjustRange on the host
//                gives scale and zero point
//   dequantize:  x = scale * (q - zero_point), q uint8 or int32
// The product and the sum are rounded separately, as the C++ expressions are.
#include <cfloat>

#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256)
quantize_f32_u8_kernel(const float *__restrict__ in, uint8_t *__restrict__ out, int64_t size, int vec4,
                       float recip_scale, float zero_point) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t done = 0;
  if (vec4) {
    const int64_t n4 = size >> 2;
    const float4 *in4 = reinterpret_cast<const float4 *>(in);
    uint32_t *out4 = reinterpret_cast<uint32_t *>(out);
    for (int64_t i = t0; i < n4; i += stride) {
      const float4 v = __ldg(in4 + i);
      const uint32_t q0 = mb_saturate_round_u8(__fadd_rn(zero_point, __fmul_rn(recip_scale, v.x)));
      const uint32_t q1 = mb_saturate_round_u8(__fadd_rn(zero_point, __fmul_rn(recip_scale, v.y)));
      const uint32_t q2 = mb_saturate_round_u8(__fadd_rn(zero_point, __fmul_rn(recip_scale, v.z)));
      const uint32_t q3 = mb_saturate_round_u8(__fadd_rn(zero_point, __fmul_rn(recip_scale, v.w)));
      out4[i] = q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
    }
    done = n4 << 2;
  }
  for (int64_t i = done + t0; i < size; i += stride)
    out[i] = static_cast<uint8_t>(mb_saturate_round_u8(__fadd_rn(zero_point, __fmul_rn(recip_scale, in[i]))));
}

template <typename Q>
__global__ void __launch_bounds__(256)
dequantize_kernel(const Q *__restrict__ in, float *__restrict__ out, int64_t size, float scale, int32_t zero_point) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < size; i += stride)
    out[i] = __fmul_rn(scale, static_cast<float>(static_cast<int32_t>(in[i]) - zero_point));
}

// min and max over the tensor; one atomic pair per warp on the order-preserving integer image
// of the floats.
__device__ __forceinline__ int32_t float_to_ordered(float f) {
  const int32_t i = __float_as_int(f);
  return i >= 0 ? i : i ^ 0x7fffffff;
}

__global__ void __launch_bounds__(256)
minmax_f32_kernel(const float *__restrict__ in, int64_t size, int32_t *__restrict__ ordered_min_max) {
  float mn = FLT_MAX, mx = -FLT_MAX;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < size; i += stride) {
    const float v = __ldg(in + i);
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMin(ordered_min_max, float_to_ordered(mn));
    atomicMax(ordered_min_max + 1, float_to_ordered(mx));
  }
}

// counts[clamp(int((x - min_v) / bin_v), 0, bins - 1)]++ with the division and subtraction
// rounded as the host's float arithmetic rounds them; a block collects in shared memory first.
__global__ void __launch_bounds__(256) histogram_f32_kernel(const float *__restrict__ in, int64_t size,
                                                            float min_v, float bin_v, int bins,
                                                            int32_t *__restrict__ counts) {
  extern __shared__ int32_t local[];
  for (int i = threadIdx.x; i < bins; i += blockDim.x) local[i] = 0;
  __syncthreads();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < size; i += stride) {
    const float q = __fdiv_rn(__fsub_rn(__ldg(in + i), min_v), bin_v);
    int index = q >= static_cast<float>(bins) ? bins - 1 : static_cast<int>(q);  // NaN -> 0
    index = min(bins - 1, max(0, index));
    atomicAdd(local + index, 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < bins; i += blockDim.x)
    if (local[i] != 0) atomicAdd(counts + i, local[i]);
}

static unsigned stream_grid(const mb_context *ctx, int64_t work_items) {
  const int64_t blocks = ceil_div64(work_items, 256);
  return static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(blocks, 16ll * ctx->num_sms)));
}

static float ordered_to_float(int32_t i) {
  const int32_t b = i >= 0 ? i : i ^ 0x7fffffff;
  float f;
  memcpy(&f, &b, 4);
  return f;
}

}  // namespace

extern "C" {

int mb_quantize_f32_u8(mb_context *ctx, const float *in, uint8_t *out, int64_t size, float scale,
                       int32_t zero_point) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (size < 0 || !(scale > 0.f)) return mb_fail(ctx, MB_INVALID_ARGS, "mb_quantize_f32_u8: bad size or scale");
  if (size == 0) return MB_SUCCESS;
  if (in == nullptr || out == nullptr) return mb_fail(ctx, MB_INVALID_ARGS, "mb_quantize_f32_u8: null operand");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  const int vec4 = (reinterpret_cast<uintptr_t>(in) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 3u) == 0;
  const float recip_scale = 1 / scale;
  quantize_f32_u8_kernel<<<stream_grid(ctx, vec4 ? size / 4 + 1 : size), 256, 0, ctx->stream>>>(
      in, out, size, vec4, recip_scale, static_cast<float>(zero_point));
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

int mb_dequantize_f32(mb_context *ctx, const void *in, int in_is_int32, float *out, int64_t size, float scale,
                      int32_t zero_point) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (size < 0) return mb_fail(ctx, MB_INVALID_ARGS, "mb_dequantize_f32: negative size");
  if (size == 0) return MB_SUCCESS;
  if (in == nullptr || out == nullptr) return mb_fail(ctx, MB_INVALID_ARGS, "mb_dequantize_f32: null operand");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  const unsigned grid = stream_grid(ctx, size);
  if (in_is_int32)
    dequantize_kernel<int32_t><<<grid, 256, 0, ctx->stream>>>(static_cast<const int32_t *>(in), out, size, scale,
                                                              zero_point);
  else
    dequantize_kernel<uint8_t><<<grid, 256, 0, ctx->stream>>>(static_cast<const uint8_t *>(in), out, size, scale,
                                                              zero_point);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

int mb_minmax_f32(mb_context *ctx, const float *in, int64_t size, float *host_min, float *host_max) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (size < 0 || host_min == nullptr || host_max == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_minmax_f32: bad argument");
  *host_min = FLT_MAX;
  *host_max = -FLT_MAX;
  if (size == 0) return MB_SUCCESS;
  if (in == nullptr) return mb_fail(ctx, MB_INVALID_ARGS, "mb_minmax_f32: null operand");
  if (ctx->capturing)
    return mb_fail(ctx, MB_RUNTIME_ERROR, "mb_minmax_f32 reads its result on the host: not inside a graph capture");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  int32_t *cell = nullptr;
  MB_RETURN_IF_ERROR(mb_scratch(ctx, 8, reinterpret_cast<void **>(&cell)));
  // start values: the ordered images of numeric_limits<float>::max() and lowest()
  static const int32_t kInit[2] = {0x7f7fffff, static_cast<int32_t>(0xff7fffffu) ^ 0x7fffffff};
  MB_CUDA(ctx, cudaMemcpyAsync(cell, kInit, 8, cudaMemcpyHostToDevice, ctx->stream));
  minmax_f32_kernel<<<stream_grid(ctx, size), 256, 0, ctx->stream>>>(in, size, cell);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  int32_t host[2];
  MB_CUDA(ctx, cudaMemcpyAsync(host, cell, 8, cudaMemcpyDeviceToHost, ctx->stream));
  MB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  *host_min = ordered_to_float(host[0]);
  *host_max = ordered_to_float(host[1]);
  return MB_SUCCESS;
}

int mb_histogram_f32(mb_context *ctx, const float *in, int64_t size, float min_v, float max_v, int bins,
                     int32_t *host_counts) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (size < 0 || bins < 1 || bins > 8192 || host_counts == nullptr || !(max_v > min_v))
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_histogram_f32: bad argument");
  if (size >= (1ll << 31)) return mb_fail(ctx, MB_UNSUPPORTED, "mb_histogram_f32: more than 2^31 - 1 values");
  memset(host_counts, 0, sizeof(int32_t) * bins);
  if (size == 0) return MB_SUCCESS;
  if (in == nullptr) return mb_fail(ctx, MB_INVALID_ARGS, "mb_histogram_f32: null operand");
  if (ctx->capturing)
    return mb_fail(ctx, MB_RUNTIME_ERROR, "mb_histogram_f32 reads its result on the host: not inside a graph capture");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  int32_t *counts = nullptr;
  MB_RETURN_IF_ERROR(mb_scratch(ctx, sizeof(int32_t) * bins, reinterpret_cast<void **>(&counts)));
  MB_CUDA(ctx, cudaMemsetAsync(counts, 0, sizeof(int32_t) * bins, ctx->stream));
  const float bin_v = (max_v - min_v) / static_cast<float>(bins);
  histogram_f32_kernel<<<stream_grid(ctx, size), 256, sizeof(int32_t) * bins, ctx->stream>>>(in, size, min_v, bin_v,
                                                                                            bins, counts);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  MB_CUDA(ctx, cudaMemcpyAsync(host_counts, counts, sizeof(int32_t) * bins, cudaMemcpyDeviceToHost, ctx->stream));
  MB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return MB_SUCCESS;
}

}  // extern "C"
