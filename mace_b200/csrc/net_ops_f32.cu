// fp32 operators that sit between the convolutions of a float network and keep its
// activations on the device: pooling (NCHW), element-wise binary ops, standalone
// activation and softmax.  All of them are bandwidth-bound streaming kernels.
//
// Reference behaviour:
//   pooling      PoolingOp<RT_CPU,float>::MaxPooling / AvgPooling (mace/ops/pooling.cc:128-240):
//                MAX starts from numeric_limits<float>::lowest() and takes the in-bounds taps;
//                AVG sums the in-bounds taps in (fh, fw) order and divides by their count.
//   eltwise      TensorEltwise / TensorScalarEltwise (mace/ops/eltwise.cc:419-700)
//   activation   ref::Activation (mace/ops/ref/activation.cc:61-88)
//   softmax      SoftmaxOp<RT_CPU,float>::RunForNCHW / RunForNHWC (mace/ops/softmax.cc:76-290):
//                max, exp(x - max), sum in class order, divide, optional log.
#include <cfloat>

#include "common.cuh"

namespace {

struct PoolF32Params {
  const float *in;
  float *out;
  int H, W, KH, KW, sh, sw, dh, dw, pad_t, pad_l, Ho, Wo;
  int64_t total;  // N * C * Ho * Wo
};

// One thread per output value; threads of a warp walk along a row, so the taps of neighbouring
// outputs fall into the same cache lines.
template <bool IS_MAX>
__global__ void __launch_bounds__(256) pooling_f32_kernel(const PoolF32Params p) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= p.total) return;
  const int w = static_cast<int>(tid % p.Wo);
  const int64_t r = tid / p.Wo;
  const int h = static_cast<int>(r % p.Ho);
  const int64_t plane = r / p.Ho;  // n * C + c
  const float *ip = p.in + plane * p.H * p.W;
  const int ih0 = h * p.sh - p.pad_t, iw0 = w * p.sw - p.pad_l;
  float res = IS_MAX ? -FLT_MAX : 0.f;
  int count = 0;
  for (int fh = 0; fh < p.KH; ++fh) {
    const int ih = ih0 + fh * p.dh;
    if (ih < 0 || ih >= p.H) continue;
    for (int fw = 0; fw < p.KW; ++fw) {
      const int iw = iw0 + fw * p.dw;
      if (iw < 0 || iw >= p.W) continue;
      const float v = __ldg(ip + ih * p.W + iw);
      if (IS_MAX) res = fmaxf(res, v);
      else res += v;
      ++count;
    }
  }
  if (!IS_MAX) res = count > 0 ? res / static_cast<float>(count) : 0.f;
  p.out[tid] = res;
}

// The same for the common "3x3 window, stride 2, no dilation" max pool on rows whose length is
// a multiple of 4 with no left padding: a thread produces four neighbouring outputs of a row
// from nine input columns, fetched per input row as two 128-bit loads and one scalar
// (9 loads for 4 outputs instead of 36).  Taps right of the image are skipped as above.
__global__ void __launch_bounds__(256) maxpool3x3s2_f32_kernel(const PoolF32Params p) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int wq = (p.Wo + 3) >> 2;
  if (tid >= p.total) return;  // total = planes * Ho * wq here
  const int q = static_cast<int>(tid % wq);
  const int64_t r = tid / wq;
  const int h = static_cast<int>(r % p.Ho);
  const int64_t plane = r / p.Ho;
  const float *ip = p.in + plane * p.H * p.W;
  const int w0 = q * 4, iw0 = w0 * 2;  // pad_l == 0
  float o[4] = {-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX};
#pragma unroll
  for (int fh = 0; fh < 3; ++fh) {
    const int ih = h * 2 - p.pad_t + fh;
    if (ih < 0 || ih >= p.H) continue;
    const float *row = ip + static_cast<int64_t>(ih) * p.W + iw0;
    float c[9];
    if (iw0 + 8 < p.W) {
      const float4 a = __ldg(reinterpret_cast<const float4 *>(row));
      const float4 b = __ldg(reinterpret_cast<const float4 *>(row) + 1);
      c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w; c[4] = b.x; c[5] = b.y; c[6] = b.z; c[7] = b.w;
      c[8] = __ldg(row + 8);
    } else {
#pragma unroll
      for (int j = 0; j < 9; ++j) c[j] = iw0 + j < p.W ? __ldg(row + j) : -FLT_MAX;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = fmaxf(o[k], fmaxf(c[2 * k], fmaxf(c[2 * k + 1], c[2 * k + 2])));
  }
  float *op = p.out + (plane * p.Ho + h) * p.Wo + w0;
  if (w0 + 3 < p.Wo && (p.Wo & 3) == 0) {
    *reinterpret_cast<float4 *>(op) = make_float4(o[0], o[1], o[2], o[3]);
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k)
      if (w0 + k < p.Wo) op[k] = o[k];
  }
}

// Element-wise binary op codes are ops::EltwiseType values (mace/ops/common/eltwise_type.h:21-38).
enum : int { ELT_SUM = 0, ELT_SUB = 1, ELT_PROD = 2, ELT_DIV = 3, ELT_MIN = 4, ELT_MAX = 5, ELT_NEG = 6,
             ELT_ABS = 7, ELT_SQR_DIFF = 8, ELT_CLIP = 12 };

struct EltParams {
  const float *in0, *in1;  // in1 null: the scalar is the second operand
  float *out;
  int64_t size;
  float scalar, c0, c1;
  int has_coeff, swapped;
  int act;  // activation applied to the result (0: none)
  float max_limit, coef;
};

template <int TYPE>
__device__ __forceinline__ float elt_op(float a, float b, const EltParams &p) {
  switch (TYPE) {
    case ELT_SUM:
      // products and sum rounded separately, as the C++ expression a * c0 + b * c1 is
      return p.has_coeff ? __fadd_rn(__fmul_rn(a, p.c0), __fmul_rn(b, p.c1)) : a + b;
    case ELT_SUB: return p.swapped ? b - a : a - b;
    case ELT_PROD: return a * b;
    case ELT_DIV: return p.swapped ? __fdiv_rn(b, a) : __fdiv_rn(a, b);
    case ELT_MIN: return fminf(a, b);
    case ELT_MAX: return fmaxf(a, b);
    case ELT_NEG: return -a;
    case ELT_ABS: return fabsf(a);
    case ELT_SQR_DIFF: { const float d = a - b; return d * d; }
    case ELT_CLIP: return fmaxf(p.c0, fminf(p.c1, a));
    default: return a;
  }
}

template <int TYPE>
__device__ __forceinline__ float elt_apply(float a, float b, const EltParams &p) {
  return mb_activate(elt_op<TYPE>(a, b, p), p.act, p.max_limit, p.coef);
}

template <int TYPE>
__global__ void __launch_bounds__(256) eltwise_f32_kernel(const EltParams p, int vec4) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (vec4) {
    const int64_t n4 = p.size >> 2;
    const float4 *a4 = reinterpret_cast<const float4 *>(p.in0);
    const float4 *b4 = reinterpret_cast<const float4 *>(p.in1);
    float4 *o4 = reinterpret_cast<float4 *>(p.out);
    for (int64_t i = t0; i < n4; i += stride) {
      const float4 a = __ldg(a4 + i);
      const float4 b = b4 != nullptr ? __ldg(b4 + i) : make_float4(p.scalar, p.scalar, p.scalar, p.scalar);
      float4 o;
      o.x = elt_apply<TYPE>(a.x, b.x, p); o.y = elt_apply<TYPE>(a.y, b.y, p);
      o.z = elt_apply<TYPE>(a.z, b.z, p); o.w = elt_apply<TYPE>(a.w, b.w, p);
      o4[i] = o;
    }
    for (int64_t i = (n4 << 2) + t0; i < p.size; i += stride)
      p.out[i] = elt_apply<TYPE>(p.in0[i], p.in1 != nullptr ? p.in1[i] : p.scalar, p);
  } else {
    for (int64_t i = t0; i < p.size; i += stride)
      p.out[i] = elt_apply<TYPE>(p.in0[i], p.in1 != nullptr ? p.in1[i] : p.scalar, p);
  }
}

__global__ void __launch_bounds__(256)
activation_f32_kernel(const float *__restrict__ in, float *__restrict__ out, int64_t size, int vec4,
                      int act, float max_limit, float coef) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t t0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t done = 0;
  if (vec4) {
    const int64_t n4 = size >> 2;
    const float4 *a4 = reinterpret_cast<const float4 *>(in);
    float4 *o4 = reinterpret_cast<float4 *>(out);
    for (int64_t i = t0; i < n4; i += stride) {
      float4 a = __ldg(a4 + i);
      a.x = mb_activate(a.x, act, max_limit, coef); a.y = mb_activate(a.y, act, max_limit, coef);
      a.z = mb_activate(a.z, act, max_limit, coef); a.w = mb_activate(a.w, act, max_limit, coef);
      o4[i] = a;
    }
    done = n4 << 2;
  }
  for (int64_t i = done + t0; i < size; i += stride) out[i] = mb_activate(in[i], act, max_limit, coef);
}

// One warp per (outer, inner) position; the classes are strided by `inner`.  The sum runs over
// the lanes' partial sums instead of class order (difference: rounding of the last bits).
__global__ void __launch_bounds__(256)
softmax_f32_kernel(const float *__restrict__ in, float *__restrict__ out, int64_t positions,
                   int64_t classes, int64_t inner, int use_log) {
  const int lane = threadIdx.x & 31;
  const int64_t pos = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (pos >= positions) return;
  const int64_t base = (pos / inner) * classes * inner + pos % inner;
  float mx = -FLT_MAX;
  for (int64_t c = lane; c < classes; c += 32) mx = fmaxf(mx, __ldg(in + base + c * inner));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int64_t c = lane; c < classes; c += 32) {
    const float e = expf(__ldg(in + base + c * inner) - mx);
    out[base + c * inner] = e;
    sum += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  for (int64_t c = lane; c < classes; c += 32) {
    const float v = __fdiv_rn(out[base + c * inner], sum);
    out[base + c * inner] = use_log ? logf(v) : v;
  }
}

static unsigned stream_grid(const mb_context *ctx, int64_t work_items) {
  const int64_t blocks = ceil_div64(work_items, 256);
  return static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(blocks, 16ll * ctx->num_sms)));
}

template <int TYPE>
static void launch_eltwise(mb_context *ctx, const EltParams &p, int vec4) {
  eltwise_f32_kernel<TYPE><<<stream_grid(ctx, vec4 ? p.size / 4 + 1 : p.size), 256, 0, ctx->stream>>>(p, vec4);
}

// out[p][ho][wo] = in[p][ho * sh][wo * sw] over N * C planes: the pixels a 1x1 convolution with
// strides (sh, sw) reads, gathered once so that several such convolutions of one tensor (a
// residual block's shortcut and its first convolution) can run as plain 1x1 convolutions on
// the compact copy.  One thread per output value, grid-stride; writes are contiguous.
__global__ void __launch_bounds__(256)
subsample_f32_kernel(const float *__restrict__ in, float *__restrict__ out, int64_t total, int H, int W, int sh,
                     int sw, int Ho, int Wo) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t plane_out = static_cast<int64_t>(Ho) * Wo, plane_in = static_cast<int64_t>(H) * W;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t pl = i / plane_out;
    const int rem = static_cast<int>(i - pl * plane_out);
    const int ho = rem / Wo, wo = rem - ho * Wo;
    out[i] = __ldg(in + pl * plane_in + static_cast<int64_t>(ho) * sh * W + wo * sw);
  }
}

}  // namespace

extern "C" {

int mb_pooling_f32_nchw(mb_context *ctx, const float *in, float *out, int64_t N, int64_t C, int64_t H,
                        int64_t W, int64_t KH, int64_t KW, int stride_h, int stride_w, int dil_h,
                        int dil_w, int pad_top, int pad_left, int64_t Ho, int64_t Wo, int pooling_type) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (N < 0 || C < 0 || H < 1 || W < 1 || KH < 1 || KW < 1 || stride_h < 1 || stride_w < 1 || dil_h < 1 ||
      dil_w < 1 || pad_top < 0 || pad_left < 0 || Ho < 0 || Wo < 0)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_pooling_f32_nchw: bad shape argument");
  if (pooling_type != 1 && pooling_type != 2)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_pooling_f32_nchw: pooling type %d (1 AVG, 2 MAX)", pooling_type);
  if (N == 0 || C == 0 || Ho == 0 || Wo == 0) return MB_SUCCESS;
  if (in == nullptr || out == nullptr) return mb_fail(ctx, MB_INVALID_ARGS, "mb_pooling_f32_nchw: null operand");
  if (H >= (1 << 30) / W || N * C * Ho * Wo >= (1ll << 40))
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_pooling_f32_nchw: tensor too large");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  PoolF32Params p;
  p.in = in; p.out = out;
  p.H = static_cast<int>(H); p.W = static_cast<int>(W); p.KH = static_cast<int>(KH); p.KW = static_cast<int>(KW);
  p.sh = stride_h; p.sw = stride_w; p.dh = dil_h; p.dw = dil_w; p.pad_t = pad_top; p.pad_l = pad_left;
  p.Ho = static_cast<int>(Ho); p.Wo = static_cast<int>(Wo);
  p.total = N * C * Ho * Wo;
  if (pooling_type == 2 && KH == 3 && KW == 3 && stride_h == 2 && stride_w == 2 && dil_h == 1 && dil_w == 1 &&
      pad_left == 0 && W % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
    p.total = N * C * Ho * ((Wo + 3) / 4);
    maxpool3x3s2_f32_kernel<<<static_cast<unsigned>(ceil_div64(p.total, 256)), 256, 0, ctx->stream>>>(p);
    MB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
    return MB_SUCCESS;
  }
  const unsigned grid = static_cast<unsigned>(ceil_div64(p.total, 256));
  if (pooling_type == 2) pooling_f32_kernel<true><<<grid, 256, 0, ctx->stream>>>(p);
  else pooling_f32_kernel<false><<<grid, 256, 0, ctx->stream>>>(p);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

int mb_eltwise_act_f32(mb_context *ctx, const float *in0, const float *in1, float *out, int64_t size, int type,
                       float scalar_input, int has_coeff, float coeff0, float coeff1, int swapped,
                       int activation, float max_limit, float coefficient) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (size < 0) return mb_fail(ctx, MB_INVALID_ARGS, "mb_eltwise_f32: negative size");
  if (!(activation == 0 || activation == 1 || activation == 2 || activation == 6))
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_eltwise_act_f32: activation %d is not built for this runtime", activation);
  if (size == 0) return MB_SUCCESS;
  if (in0 == nullptr || out == nullptr) return mb_fail(ctx, MB_INVALID_ARGS, "mb_eltwise_f32: null operand");
  if (type == ELT_CLIP && !(has_coeff && coeff0 < coeff1))
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_eltwise_f32: Clip's min/max values are not correct.");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  EltParams p;
  p.in0 = in0; p.in1 = in1; p.out = out; p.size = size; p.scalar = scalar_input;
  // a swapped SUM swaps the coefficients (mace/ops/eltwise.cc:437-440)
  p.c0 = (swapped && type == ELT_SUM) ? coeff1 : coeff0;
  p.c1 = (swapped && type == ELT_SUM) ? coeff0 : coeff1;
  p.has_coeff = has_coeff; p.swapped = swapped;
  p.act = activation; p.max_limit = max_limit; p.coef = coefficient;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(in0) | reinterpret_cast<uintptr_t>(in1) |
                         reinterpret_cast<uintptr_t>(out);
  const int vec4 = (bits & 15u) == 0;
  switch (type) {
    case ELT_SUM: launch_eltwise<ELT_SUM>(ctx, p, vec4); break;
    case ELT_SUB: launch_eltwise<ELT_SUB>(ctx, p, vec4); break;
    case ELT_PROD: launch_eltwise<ELT_PROD>(ctx, p, vec4); break;
    case ELT_DIV: launch_eltwise<ELT_DIV>(ctx, p, vec4); break;
    case ELT_MIN: launch_eltwise<ELT_MIN>(ctx, p, vec4); break;
    case ELT_MAX: launch_eltwise<ELT_MAX>(ctx, p, vec4); break;
    case ELT_NEG: launch_eltwise<ELT_NEG>(ctx, p, vec4); break;
    case ELT_ABS: launch_eltwise<ELT_ABS>(ctx, p, vec4); break;
    case ELT_SQR_DIFF: launch_eltwise<ELT_SQR_DIFF>(ctx, p, vec4); break;
    case ELT_CLIP: launch_eltwise<ELT_CLIP>(ctx, p, vec4); break;
    default: return mb_fail(ctx, MB_UNSUPPORTED, "mb_eltwise_f32: type %d is not built for this runtime", type);
  }
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

int mb_eltwise_f32(mb_context *ctx, const float *in0, const float *in1, float *out, int64_t size, int type,
                   float scalar_input, int has_coeff, float coeff0, float coeff1, int swapped) {
  return mb_eltwise_act_f32(ctx, in0, in1, out, size, type, scalar_input, has_coeff, coeff0, coeff1, swapped, 0,
                            0.f, 0.f);
}

int mb_activation_f32(mb_context *ctx, const float *in, float *out, int64_t size, int activation,
                      float max_limit, float coefficient) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (size < 0) return mb_fail(ctx, MB_INVALID_ARGS, "mb_activation_f32: negative size");
  if (!(activation == 0 || activation == 1 || activation == 2 || activation == 6))
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_activation_f32: activation %d is not built for this runtime",
                   activation);
  if (size == 0) return MB_SUCCESS;
  if (in == nullptr || out == nullptr) return mb_fail(ctx, MB_INVALID_ARGS, "mb_activation_f32: null operand");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  const int vec4 = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
  activation_f32_kernel<<<stream_grid(ctx, vec4 ? size / 4 + 1 : size), 256, 0, ctx->stream>>>(
      in, out, size, vec4, activation, max_limit, coefficient);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

int mb_softmax_f32(mb_context *ctx, const float *in, float *out, int64_t outer, int64_t classes, int64_t inner,
                   int use_log) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (outer < 0 || classes < 0 || inner < 0) return mb_fail(ctx, MB_INVALID_ARGS, "mb_softmax_f32: negative size");
  if (outer == 0 || classes == 0 || inner == 0) return MB_SUCCESS;
  if (in == nullptr || out == nullptr) return mb_fail(ctx, MB_INVALID_ARGS, "mb_softmax_f32: null operand");
  const int64_t positions = outer * inner;
  if (ceil_div64(positions, 8) >= (1ll << 31)) return mb_fail(ctx, MB_UNSUPPORTED, "mb_softmax_f32: tensor too large");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  softmax_f32_kernel<<<static_cast<unsigned>(ceil_div64(positions, 8)), 256, 0, ctx->stream>>>(
      in, out, positions, classes, inner, use_log);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

int mb_subsample_f32_nchw(mb_context *ctx, const float *in, float *out, int64_t planes, int64_t H, int64_t W,
                          int stride_h, int stride_w) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (planes < 0 || H < 0 || W < 0 || stride_h < 1 || stride_w < 1 || H > INT32_MAX || W > INT32_MAX)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_subsample_f32_nchw: bad extents or strides");
  const int64_t Ho = ceil_div64(H, stride_h), Wo = ceil_div64(W, stride_w);
  const int64_t total = planes * Ho * Wo;
  if (total == 0) return MB_SUCCESS;
  if (in == nullptr || out == nullptr || in == out)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_subsample_f32_nchw: null or aliased buffers");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  subsample_f32_kernel<<<stream_grid(ctx, total), 256, 0, ctx->stream>>>(in, out, total, static_cast<int>(H),
                                                                         static_cast<int>(W), stride_h, stride_w,
                                                                         static_cast<int>(Ho), static_cast<int>(Wo));
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

}  // extern "C"
