// uint8 average pooling, NHWC.
//
// Reference behaviour: PoolingOp<RT_CPU,uint8_t> with AVG
// (mace/ops/pooling.cc:638-871): for each output pixel the window is clipped
// to the image, block = clipped height * width, and every channel gets
// (sum + block / 2) / block in unsigned 32-bit arithmetic.  The output keeps
// the input's scale and zero point (:651-653).
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256)
avgpool_u8_kernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out, int N, int H, int W,
                  int C, int KH, int KW, int sh, int sw, int pad_top, int pad_left, int Ho, int Wo) {
  const int64_t total = static_cast<int64_t>(N) * Ho * Wo * C;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int c = static_cast<int>(tid % C);
  int64_t r = tid / C;
  const int wo = static_cast<int>(r % Wo);
  r /= Wo;
  const int ho = static_cast<int>(r % Ho);
  const int n = static_cast<int>(r / Ho);
  const int hb = ho * sh - pad_top, wb = wo * sw - pad_left;
  const int h0 = max(0, hb), w0 = max(0, wb);
  const int h1 = min(H, hb + KH), w1 = min(W, wb + KW);
  const uint32_t block = static_cast<uint32_t>((h1 - h0) * (w1 - w0));
  uint32_t sum = 0;
  for (int h = h0; h < h1; ++h)
    for (int w = w0; w < w1; ++w)
      sum += in[((static_cast<int64_t>(n) * H + h) * W + w) * C + c];
  out[tid] = static_cast<uint8_t>((sum + block / 2) / block);
}

// Four adjacent channels per thread (one 32-bit word per pixel), all loads of a window row in
// flight together; C % 4 == 0 and 4-byte aligned tensors.
__global__ void __launch_bounds__(128)
avgpool_u8_c4_kernel(const uint8_t *__restrict__ in, uint8_t *__restrict__ out, int N, int H, int W,
                     int C, int KH, int KW, int sh, int sw, int pad_top, int pad_left, int Ho, int Wo) {
  mb_grid_dep_launch();
  mb_grid_dep_wait();
  const int groups = C >> 2;
  const unsigned total = static_cast<unsigned>(N) * Ho * Wo * groups;
  const unsigned tid = blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int g = tid % groups;
  unsigned r = tid / groups;
  const int wo = r % Wo;
  r /= Wo;
  const int ho = r % Ho;
  const int n = r / Ho;
  const int hb = ho * sh - pad_top, wb = wo * sw - pad_left;
  const int h0 = max(0, hb), w0 = max(0, wb);
  const int h1 = min(H, hb + KH), w1 = min(W, wb + KW);
  const uint32_t block = static_cast<uint32_t>((h1 - h0) * (w1 - w0));
  uint32_t s0 = 0, s1 = 0, s2 = 0, s3 = 0;
  const uint8_t *base = in + (static_cast<int64_t>(n) * H * W) * C + g * 4;
  if (h1 - h0 == 7 && w1 - w0 == 7) {
    // the 7x7 window of a global pooling layer: all 49 loads requested before any is used
    uint32_t v[49];
#pragma unroll
    for (int i = 0; i < 49; ++i)
      v[i] = __ldg(reinterpret_cast<const uint32_t *>(
          base + (static_cast<int64_t>(h0 + i / 7) * W + (w0 + i % 7)) * C));
#pragma unroll
    for (int i = 0; i < 49; ++i) {
      s0 = __dp4a(v[i], 0x00000001u, s0);
      s1 = __dp4a(v[i], 0x00000100u, s1);
      s2 = __dp4a(v[i], 0x00010000u, s2);
      s3 = __dp4a(v[i], 0x01000000u, s3);
    }
  } else
  for (int h = h0; h < h1; ++h) {
    const uint8_t *row = base + static_cast<int64_t>(h) * W * C;
#pragma unroll 8
    for (int w = w0; w < w1; ++w) {
      const uint32_t v = __ldg(reinterpret_cast<const uint32_t *>(row + static_cast<int64_t>(w) * C));
      s0 = __dp4a(v, 0x00000001u, s0);
      s1 = __dp4a(v, 0x00000100u, s1);
      s2 = __dp4a(v, 0x00010000u, s2);
      s3 = __dp4a(v, 0x01000000u, s3);
    }
  }
  const uint32_t half = block / 2;
  const uint32_t o = ((s0 + half) / block) | (((s1 + half) / block) << 8) | (((s2 + half) / block) << 16) |
                     (((s3 + half) / block) << 24);
  *reinterpret_cast<uint32_t *>(out + static_cast<int64_t>(tid) * 4) = o;
}

}  // namespace

extern "C" int mb_avgpool_u8_nhwc(mb_context *ctx, const uint8_t *in, uint8_t *out, int64_t N,
                                  int64_t H, int64_t W, int64_t C, int64_t KH, int64_t KW,
                                  int stride_h, int stride_w, int pad_top, int pad_left,
                                  int64_t Ho, int64_t Wo) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (N < 0 || H < 1 || W < 1 || C < 1 || KH < 1 || KW < 1 || Ho < 0 || Wo < 0 || stride_h < 1 ||
      stride_w < 1 || pad_top < 0 || pad_left < 0)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_avgpool_u8_nhwc: bad shape argument");
  if (N == 0 || Ho == 0 || Wo == 0) return MB_SUCCESS;
  if (in == nullptr || out == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_avgpool_u8_nhwc: null operand");
  // every window must overlap the image (the reference checks block_size > 0)
  if ((Ho - 1) * stride_h - pad_top >= H || (Wo - 1) * stride_w - pad_left >= W ||
      pad_top >= KH || pad_left >= KW)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_avgpool_u8_nhwc: a window lies outside the image");
  const int64_t total = N * Ho * Wo * C;
  if (ceil_div64(total, 256) > 0x7fffffffll || N * H * W * C >= (1ll << 40))
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_avgpool_u8_nhwc: tensor too large");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  if (C % 4 == 0 && total / 4 < (1ll << 31) &&
      ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 3u) == 0) {
    MB_CUDA(ctx, mb_launch_chained(ctx, avgpool_u8_c4_kernel, dim3(static_cast<unsigned>(ceil_div64(total / 4, 128))),
                                   dim3(128), 0, in, out, static_cast<int>(N), static_cast<int>(H),
                                   static_cast<int>(W), static_cast<int>(C), static_cast<int>(KH),
                                   static_cast<int>(KW), stride_h, stride_w, pad_top, pad_left,
                                   static_cast<int>(Ho), static_cast<int>(Wo)));
    MB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
    return MB_SUCCESS;
  }
  avgpool_u8_kernel<<<static_cast<unsigned>(ceil_div64(total, 256)), 256, 0, ctx->stream>>>(
      in, out, static_cast<int>(N), static_cast<int>(H), static_cast<int>(W), static_cast<int>(C),
      static_cast<int>(KH), static_cast<int>(KW), stride_h, stride_w, pad_top, pad_left,
      static_cast<int>(Ho), static_cast<int>(Wo));
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}
