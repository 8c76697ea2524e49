// uint8 depthwise convolution, NHWC input, HWIM filter, NHWC output.
//
// Reference behaviour: DepthwiseConv2dOp<RT_CPU,uint8_t>::Run
// (mace/ops/depthwise_conv2d.cc:152-250): int32 accumulation of
// (in - zp_in) * (f - zp_f) over the taps that fall inside the image, + bias,
// fixed-point requantization (same primitives as the GEMM output pipeline),
// + zp_out, clamp to [0,255]; and its dilated fallback DepthwiseConv2dGeneral
// (:252-320), which requantizes with int(round(acc * multiplier_float)).
//
// Data layout: channels are innermost, so one warp reads 128 consecutive
// channel bytes of a pixel in one transaction.  Each thread owns 4 adjacent
// channels (one 32-bit word per tap) and a short strip of output pixels along
// W; the filter taps of its channels stay in registers for the whole strip.
#include "common.cuh"

namespace {

struct DwParams {
  const uint8_t *in, *filter;
  const int32_t *bias;
  uint8_t *out;
  int N, H, W, C, mult_ch, KH, KW, stride_h, stride_w, dil_h, dil_w, pad_top, pad_left, Ho, Wo;
  int32_t zp_in, zp_f, zp_out;
  mb_requant_params rq;
  int use_float;
  float mult_f;
};

__device__ __forceinline__ uint32_t dw_requant(int32_t acc, const DwParams &p) {
  if (p.use_float) {
    // sum = static_cast<int32_t>(std::round(sum * multiplier)); sum += zp_out
    const int32_t v =
        static_cast<int32_t>(roundf(__fmul_rn(static_cast<float>(acc), p.mult_f))) + p.zp_out;
    return static_cast<uint32_t>(min(255, max(0, v)));
  }
  return mb_requant_fast(acc, p.rq);
}

// dp2a with signed 16-bit halves in `a` and UNSIGNED bytes in `b`:
//   lo: c + a.lo * b.byte0 + a.hi * b.byte1     hi: c + a.lo * b.byte2 + a.hi * b.byte3
__device__ __forceinline__ int32_t dp2a_lo_s16_u8(int32_t a, uint32_t b, int32_t c) {
  int32_t d;
  asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int32_t dp2a_hi_s16_u8(int32_t a, uint32_t b, int32_t c) {
  int32_t d;
  asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Fast path: 3x3, channel multiplier 1, dilation 1, C % 4 == 0.  A thread owns
// 4 adjacent channels (one 32-bit word per pixel) and STRIP output pixels along
// W.  One dp2a per tap and channel multiplies the raw input byte with the
// zero-point-free filter value (f - zp_f, kept as a signed 16-bit half-word;
// the other half is 0 and masks the neighbouring channel's byte), so nothing is
// unpacked.  The input zero point is folded into the start value:
//   sum (in - zp_in)(f - zp_f) = sum in (f - zp_f) - zp_in * sum (f - zp_f)
// with out-of-image taps read as zp_in, which makes them contribute zero.
template <int STRIDE, int STRIP>
__global__ void __launch_bounds__(256) dwconv3x3_u8_kernel(const DwParams p) {
  const int cgroups = p.C >> 2;
  const int strips_w = (p.Wo + STRIP - 1) / STRIP;
  const int64_t total = static_cast<int64_t>(p.N) * p.Ho * strips_w * cgroups;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int cg = static_cast<int>(tid % cgroups);
  int64_t r = tid / cgroups;
  const int sw = static_cast<int>(r % strips_w);
  r /= strips_w;
  const int ho = static_cast<int>(r % p.Ho);
  const int n = static_cast<int>(r / p.Ho);
  const int c0 = cg * 4;
  const int wo0 = sw * STRIP;

  int32_t wq[9][4];
  int32_t fsum[4] = {0, 0, 0, 0};
#pragma unroll
  for (int t = 0; t < 9; ++t) {
    const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(p.filter + t * p.C + c0));
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int32_t f = static_cast<int32_t>((w >> (8 * c)) & 0xffu) - p.zp_f;
      fsum[c] += f;
      wq[t][c] = (c & 1) ? (f << 16) : (f & 0xffff);
    }
  }
  int32_t start[4];
  {
    int32_t b4[4] = {0, 0, 0, 0};
    if (p.bias != nullptr) {
      const int4 bv = __ldg(reinterpret_cast<const int4 *>(p.bias + c0));
      b4[0] = bv.x; b4[1] = bv.y; b4[2] = bv.z; b4[3] = bv.w;
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) start[c] = b4[c] - p.zp_in * fsum[c];
  }
  int32_t acc[STRIP][4];
#pragma unroll
  for (int s = 0; s < STRIP; ++s)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[s][c] = start[c];

  constexpr int COLS = (STRIP - 1) * STRIDE + 3;  // input columns the strip touches
  const int hi0 = ho * STRIDE - p.pad_top;
  const int wi0 = wo0 * STRIDE - p.pad_left;
  const uint32_t zi4 = static_cast<uint32_t>(p.zp_in) * 0x01010101u;
  const uint8_t *in_n = p.in + static_cast<int64_t>(n) * p.H * p.W * p.C + c0;
#pragma unroll
  for (int kh = 0; kh < 3; ++kh) {
    const int hi = hi0 + kh;
    const bool row_ok = hi >= 0 && hi < p.H;
    const uint8_t *row = in_n + static_cast<int64_t>(row_ok ? hi : 0) * p.W * p.C;
    uint32_t wv[COLS];
#pragma unroll
    for (int j = 0; j < COLS; ++j) {
      const int wi = wi0 + j;
      const bool ok = row_ok && wi >= 0 && wi < p.W;
      wv[j] = ok ? __ldg(reinterpret_cast<const uint32_t *>(row + static_cast<int64_t>(wi) * p.C)) : zi4;
    }
#pragma unroll
    for (int j = 0; j < COLS; ++j) {
#pragma unroll
      for (int s = 0; s < STRIP; ++s) {
        const int kw = j - s * STRIDE;  // compile-time after unrolling
        if (kw >= 0 && kw < 3) {
          const int t = kh * 3 + kw;
          acc[s][0] = dp2a_lo_s16_u8(wq[t][0], wv[j], acc[s][0]);
          acc[s][1] = dp2a_lo_s16_u8(wq[t][1], wv[j], acc[s][1]);
          acc[s][2] = dp2a_hi_s16_u8(wq[t][2], wv[j], acc[s][2]);
          acc[s][3] = dp2a_hi_s16_u8(wq[t][3], wv[j], acc[s][3]);
        }
      }
    }
  }
  uint8_t *out_row = p.out + ((static_cast<int64_t>(n) * p.Ho + ho) * p.Wo) * p.C + c0;
#pragma unroll
  for (int s = 0; s < STRIP; ++s) {
    const int wo = wo0 + s;
    if (wo >= p.Wo) break;
    uint32_t w = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) w |= dw_requant(acc[s][c], p) << (8 * c);
    *reinterpret_cast<uint32_t *>(out_row + static_cast<int64_t>(wo) * p.C) = w;
  }
}

// General path: any filter size, stride, dilation, channel multiplier and
// channel count; one thread per output element.
__global__ void __launch_bounds__(256) dwconv_u8_general_kernel(const DwParams p) {
  const int OC = p.C * p.mult_ch;
  const int64_t total = static_cast<int64_t>(p.N) * p.Ho * p.Wo * OC;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int m = static_cast<int>(tid % OC);
  int64_t r = tid / OC;
  const int wo = static_cast<int>(r % p.Wo);
  r /= p.Wo;
  const int ho = static_cast<int>(r % p.Ho);
  const int n = static_cast<int>(r / p.Ho);
  const int c = m / p.mult_ch, o = m % p.mult_ch;
  int32_t acc = 0;
  for (int kh = 0; kh < p.KH; ++kh) {
    const int hi = ho * p.stride_h - p.pad_top + kh * p.dil_h;
    if (hi < 0 || hi >= p.H) continue;
    for (int kw = 0; kw < p.KW; ++kw) {
      const int wi = wo * p.stride_w - p.pad_left + kw * p.dil_w;
      if (wi < 0 || wi >= p.W) continue;
      const int32_t iv = p.in[((static_cast<int64_t>(n) * p.H + hi) * p.W + wi) * p.C + c];
      const int32_t fv = p.filter[((kh * p.KW + kw) * p.C + c) * p.mult_ch + o];
      acc += (iv - p.zp_in) * (fv - p.zp_f);
    }
  }
  if (p.bias != nullptr) acc += p.bias[m];
  p.out[tid] = static_cast<uint8_t>(dw_requant(acc, p));
}

}  // namespace

extern "C" int mb_dwconv_u8_nhwc(mb_context *ctx, const uint8_t *in, const uint8_t *filter,
                                 const int32_t *bias, uint8_t *out, int64_t N, int64_t H,
                                 int64_t W, int64_t C, int64_t mult_ch, int64_t KH, int64_t KW,
                                 int stride_h, int stride_w, int dil_h, int dil_w, int pad_top,
                                 int pad_left, int64_t Ho, int64_t Wo, int32_t zp_in,
                                 int32_t zp_f, int32_t multiplier, int32_t right_shift,
                                 int32_t zp_out, int use_float_multiplier, float multiplier_f) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (N < 0 || H < 1 || W < 1 || C < 1 || mult_ch < 1 || KH < 1 || KW < 1 || Ho < 0 || Wo < 0 ||
      stride_h < 1 || stride_w < 1 || dil_h < 1 || dil_w < 1 || pad_top < 0 || pad_left < 0)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_dwconv_u8_nhwc: bad shape argument");
  if (N == 0 || Ho == 0 || Wo == 0) return MB_SUCCESS;
  if (in == nullptr || filter == nullptr || out == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_dwconv_u8_nhwc: null operand");
  if (!use_float_multiplier && (multiplier <= 0 || right_shift < 0 || right_shift > 31))
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_dwconv_u8_nhwc: bad multiplier/shift");
  if (zp_out < 0 || zp_out > 255)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_dwconv_u8_nhwc: output zero point outside uint8");
  if (N * H * W * C >= (1ll << 40) || H > 65535 * 16 || W > 65535 * 16 || C > (1 << 24))
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_dwconv_u8_nhwc: tensor too large");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  DwParams p;
  p.in = in; p.filter = filter; p.bias = bias; p.out = out;
  p.N = static_cast<int>(N); p.H = static_cast<int>(H); p.W = static_cast<int>(W);
  p.C = static_cast<int>(C); p.mult_ch = static_cast<int>(mult_ch);
  p.KH = static_cast<int>(KH); p.KW = static_cast<int>(KW);
  p.stride_h = stride_h; p.stride_w = stride_w; p.dil_h = dil_h; p.dil_w = dil_w;
  p.pad_top = pad_top; p.pad_left = pad_left; p.Ho = static_cast<int>(Ho); p.Wo = static_cast<int>(Wo);
  p.zp_in = zp_in; p.zp_f = zp_f; p.zp_out = zp_out;
  p.rq = mb_make_requant(use_float_multiplier ? (1 << 30) : multiplier, use_float_multiplier ? 0 : right_shift, zp_out);
  p.use_float = use_float_multiplier; p.mult_f = multiplier_f;

  const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(filter) |
                         reinterpret_cast<uintptr_t>(out)) & 3u) == 0 &&
                       (bias == nullptr || (reinterpret_cast<uintptr_t>(bias) & 15u) == 0);
  const bool fast = KH == 3 && KW == 3 && mult_ch == 1 && dil_h == 1 && dil_w == 1 &&
                    zp_in >= 0 && zp_in <= 255 && !use_float_multiplier &&
                    stride_h == stride_w && (stride_h == 1 || stride_h == 2) && C % 4 == 0 &&
                    aligned;
  if (fast) {
    constexpr int STRIP = 4;
    const int64_t total = N * Ho * ceil_div64(Wo, STRIP) * (C / 4);
    const unsigned blocks = static_cast<unsigned>(ceil_div64(total, 256));
    if (stride_h == 1) dwconv3x3_u8_kernel<1, STRIP><<<blocks, 256, 0, ctx->stream>>>(p);
    else dwconv3x3_u8_kernel<2, STRIP><<<blocks, 256, 0, ctx->stream>>>(p);
  } else {
    const int64_t total = N * Ho * Wo * C * mult_ch;
    if (ceil_div64(total, 256) > 0x7fffffffll)
      return mb_fail(ctx, MB_UNSUPPORTED, "mb_dwconv_u8_nhwc: output too large");
    dwconv_u8_general_kernel<<<static_cast<unsigned>(ceil_div64(total, 256)), 256, 0, ctx->stream>>>(p);
  }
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}
