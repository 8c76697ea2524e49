// uint8 Conv2D, NHWC input, OHWI filter, NHWC output.
//
// Reference behaviour: Conv2dOp<RT_CPU,uint8_t>::Run (mace/ops/conv_2d.cc:
// 201-318): [im2col with the input zero point as pad value, :322-412] then a
// GEMM filter[O x depth] * patches[depth x pixels] with a per-output-channel
// int32 bias and the fixed-point output pipeline.  Padding with the zero point
// contributes (zp - zp) * w = 0, i.e. exactly the sum over in-bounds taps.
//
// Three routes:
//   1x1 stride 1      -> the NHWC tensor already is the [pixels x C] K-major
//                        GEMM operand; no copy (conv_2d.cc:279-281)
//   3x3 on 3 channels -> packed-patch dp4a kernel (MobileNet's 3x3x3 stem)
//   small depth * O   -> direct kernel, one thread per output pixel, the whole
//                        filter in shared memory
//   everything else   -> patch gather into scratch (rows padded to 16 bytes)
//                        + tensor-core GEMM
#include "common.cuh"

int mb_gemm_u8_rowmajor(mb_context *ctx, const uint8_t *A, const uint8_t *B, const int32_t *bias,
                        void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N,
                        int64_t K, bool a_mn, bool b_mn, int a_batched, int b_batched,
                        int32_t zp_a, int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c,
                        int bias_per_row);

namespace {

struct ConvParams {
  const uint8_t *in, *filter;
  const int32_t *bias;
  uint8_t *out;
  int N, H, W, C, O, KH, KW, stride_h, stride_w, pad_top, pad_left, Ho, Wo;
  int depth, depth_padded;
  int32_t zp_in, zp_f;
  mb_requant_params rq;
  int rq_variant;  // mb_requant_variant()
};

// Direct convolution: thread = one output pixel, OT output channels at a time.
// Filter (zero point removed, int16) lives in shared memory as [depth][O].
template <int OT>
__global__ void __launch_bounds__(128) conv_u8_direct_kernel(const ConvParams p) {
  extern __shared__ int16_t fsm[];  // [depth][O]
  for (int i = threadIdx.x; i < p.depth * p.O; i += blockDim.x) {
    const int d = i / p.O, o = i % p.O;
    fsm[i] = static_cast<int16_t>(static_cast<int32_t>(p.filter[o * p.depth + d]) - p.zp_f);
  }
  __syncthreads();
  const int64_t pix = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t npix = static_cast<int64_t>(p.N) * p.Ho * p.Wo;
  if (pix >= npix) return;
  const int wo = static_cast<int>(pix % p.Wo);
  const int ho = static_cast<int>((pix / p.Wo) % p.Ho);
  const int n = static_cast<int>(pix / (static_cast<int64_t>(p.Wo) * p.Ho));
  const int hi0 = ho * p.stride_h - p.pad_top, wi0 = wo * p.stride_w - p.pad_left;
  const uint8_t *in_n = p.in + static_cast<int64_t>(n) * p.H * p.W * p.C;
  uint8_t *outp = p.out + pix * p.O;
  for (int o0 = 0; o0 < p.O; o0 += OT) {
    int32_t acc[OT];
#pragma unroll
    for (int j = 0; j < OT; ++j)
      acc[j] = (p.bias != nullptr && o0 + j < p.O) ? p.bias[o0 + j] : 0;
    for (int kh = 0; kh < p.KH; ++kh) {
      const int hi = hi0 + kh;
      if (hi < 0 || hi >= p.H) continue;
      for (int kw = 0; kw < p.KW; ++kw) {
        const int wi = wi0 + kw;
        if (wi < 0 || wi >= p.W) continue;
        const uint8_t *ip = in_n + (static_cast<int64_t>(hi) * p.W + wi) * p.C;
        const int16_t *fp = fsm + ((kh * p.KW + kw) * p.C) * p.O + o0;
        for (int c = 0; c < p.C; ++c) {
          const int32_t iv = static_cast<int32_t>(__ldg(ip + c)) - p.zp_in;
#pragma unroll
          for (int j = 0; j < OT; ++j)
            if (o0 + j < p.O) acc[j] += iv * fp[c * p.O + j];
        }
      }
    }
#pragma unroll
    for (int j = 0; j < OT; ++j)
      if (o0 + j < p.O)
        outp[o0 + j] = static_cast<uint8_t>(mb_requant_fast(acc[j], p.rq));
  }
}

// First-layer style convolution (few input channels, e.g. 3x3x3): thread = one
// output pixel, all output channels.  The KH*KW*C patch bytes are packed into
// DW 32-bit words held in registers and multiplied with the raw filter bytes
// by dp4a; zero points are applied afterwards:
//   sum (in - zi)(f - zf) = sum in*f - zf * sum in - zi * sum f + depth * zi * zf
// with out-of-image taps read as zi (so they contribute zero).  The filter
// rows (zero-padded to 8 words) and the per-channel constant
//   bias - zi * sum f + depth * zi * zf
// live in shared memory and are read as broadcasts.
// All output channels of one pixel from its packed patch: four channels per step, filter
// rows read as 128-bit broadcasts.
template <int DW, int DWP, int VAR>
__device__ __forceinline__ uint32_t patch_outputs4(const uint32_t (&patch)[DW], const uint32_t *smem_w,
                                                   const int32_t *cterm, int32_t in_term,
                                                   const ConvParams &p, int o0) {
  const int4 ct = *reinterpret_cast<const int4 *>(cterm + o0);
  const int32_t c4[4] = {ct.x, ct.y, ct.z, ct.w};
  int32_t a[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 *wr = reinterpret_cast<const uint4 *>(smem_w + (o0 + j) * DWP);
    uint32_t dot = 0;
#pragma unroll
    for (int q = 0; q < DWP / 4; ++q) {
      const uint4 w4 = wr[q];
      if (q * 4 + 0 < DW) dot = __dp4a(patch[q * 4 + 0 < DW ? q * 4 + 0 : 0], w4.x, dot);
      if (q * 4 + 1 < DW) dot = __dp4a(patch[q * 4 + 1 < DW ? q * 4 + 1 : 0], w4.y, dot);
      if (q * 4 + 2 < DW) dot = __dp4a(patch[q * 4 + 2 < DW ? q * 4 + 2 : 0], w4.z, dot);
      if (q * 4 + 3 < DW) dot = __dp4a(patch[q * 4 + 3 < DW ? q * 4 + 3 : 0], w4.w, dot);
    }
    a[j] = static_cast<int32_t>(dot) + in_term + c4[j];
  }
  if (VAR >= 4) return mb_requant_pack4<VAR == 5>(a[0], a[1], a[2], a[3], p.rq);
  uint32_t b[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) b[j] = mb_requant_t<(VAR & 1) != 0, (VAR & 2) != 0>(a[j], p.rq);
  return __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
}

// All output channels of one pixel from its packed patch: four channels per step (filter rows
// and constants read as 128-bit broadcasts), sixteen per store where the channel count allows.
template <int DW, int DWP, int VAR>
__device__ __forceinline__ void patch_outputs(const uint32_t (&patch)[DW], const uint32_t *smem_w,
                                              const int32_t *cterm, int32_t in_term,
                                              const ConvParams &p, uint8_t *outp) {
  if ((p.O & 15) == 0 && (reinterpret_cast<uintptr_t>(outp) & 15u) == 0) {
    for (int o0 = 0; o0 < p.O; o0 += 16) {
      uint4 v;
      v.x = patch_outputs4<DW, DWP, VAR>(patch, smem_w, cterm, in_term, p, o0);
      v.y = patch_outputs4<DW, DWP, VAR>(patch, smem_w, cterm, in_term, p, o0 + 4);
      v.z = patch_outputs4<DW, DWP, VAR>(patch, smem_w, cterm, in_term, p, o0 + 8);
      v.w = patch_outputs4<DW, DWP, VAR>(patch, smem_w, cterm, in_term, p, o0 + 12);
      *reinterpret_cast<uint4 *>(outp + o0) = v;
    }
    return;
  }
  for (int o0 = 0; o0 < p.O; o0 += 4)
    *reinterpret_cast<uint32_t *>(outp + o0) = patch_outputs4<DW, DWP, VAR>(patch, smem_w, cterm, in_term, p, o0);
}

template <int KH, int KW, int C>
__global__ void __launch_bounds__(128) conv_u8_patch_dp4a_kernel(const ConvParams p) {
  constexpr int DEPTH = KH * KW * C;
  constexpr int DW = (DEPTH + 3) / 4;
  constexpr int DWP = (DW + 3) / 4 * 4;  // words per filter row in shared memory
  extern __shared__ uint32_t smem_w[];   // [O][DWP] filter words, then [O] constants
  int32_t *cterm = reinterpret_cast<int32_t *>(smem_w + p.O * DWP);
  mb_grid_dep_launch();
  mb_grid_dep_wait();
  for (int i = threadIdx.x; i < p.O * DWP; i += blockDim.x) {
    const int o = i / DWP, w = i % DWP;
    uint32_t v = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int d = w * 4 + b;
      if (d < DEPTH) v |= static_cast<uint32_t>(p.filter[o * DEPTH + d]) << (8 * b);
    }
    smem_w[i] = v;
  }
  for (int o = threadIdx.x; o < p.O; o += blockDim.x) {
    int32_t fs = 0;
    for (int d = 0; d < DEPTH; ++d) fs += p.filter[o * DEPTH + d];
    cterm[o] = (p.bias != nullptr ? p.bias[o] : 0) - p.zp_in * fs + DEPTH * p.zp_in * p.zp_f;
  }
  __syncthreads();
  // a block walks over several 128-pixel groups, so that packing the filter above is paid
  // once per block and not once per 128 pixels
  const int64_t npix = static_cast<int64_t>(p.N) * p.Ho * p.Wo;
  for (int64_t pix = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; pix < npix;
       pix += static_cast<int64_t>(gridDim.x) * blockDim.x) {
  const int wo = static_cast<int>(pix % p.Wo);
  const int ho = static_cast<int>((pix / p.Wo) % p.Ho);
  const int n = static_cast<int>(pix / (static_cast<int64_t>(p.Wo) * p.Ho));
  const int hi0 = ho * p.stride_h - p.pad_top, wi0 = wo * p.stride_w - p.pad_left;
  const uint8_t *in_n = p.in + static_cast<int64_t>(n) * p.H * p.W * C;
  uint32_t patch[DW];
#pragma unroll
  for (int i = 0; i < DW; ++i) patch[i] = 0;
  const uint32_t zi = static_cast<uint32_t>(p.zp_in);
  // Interior pixels of a 3x3x3 window: a window row is 9 contiguous bytes (3 pixels x 3
  // channels).  Three aligned 32-bit loads cover it (plus up to 3 bytes, which the "wi0 + 3 < W"
  // condition keeps inside the tensor), a funnel shift removes the misalignment, and the three
  // rows are spliced into the 27-byte patch at byte offsets 0, 9 and 18: 9 loads and about 20
  // logic instructions instead of 27 byte loads with their address arithmetic and merges.
  const bool interior = KH == 3 && KW == 3 && C == 3 && hi0 >= 0 && wi0 >= 0 && hi0 + 2 < p.H &&
                        wi0 + 3 < p.W && (reinterpret_cast<uintptr_t>(p.in) & 3u) == 0;
  if (interior) {
    uint32_t r[3][3];
#pragma unroll
    for (int kh = 0; kh < 3; ++kh) {
      const int64_t a = (static_cast<int64_t>(n) * p.H + hi0 + kh) * p.W * 3 + static_cast<int64_t>(wi0) * 3;
      const uint32_t *wp = reinterpret_cast<const uint32_t *>(p.in + (a & ~static_cast<int64_t>(3)));
      const uint32_t sh = (static_cast<uint32_t>(a) & 3u) * 8;
      const uint32_t w0 = __ldg(wp), w1 = __ldg(wp + 1), w2 = __ldg(wp + 2);
      r[kh][0] = __funnelshift_r(w0, w1, sh);
      r[kh][1] = __funnelshift_r(w1, w2, sh);
      r[kh][2] = (w2 >> sh) & 0xffu;  // the row's ninth byte
    }
    patch[0] = r[0][0];
    patch[1] = r[0][1];
    patch[2] = r[0][2] | (r[1][0] << 8);
    patch[3] = __funnelshift_r(r[1][0], r[1][1], 24);
    patch[4] = (r[1][1] >> 24) | (r[1][2] << 8) | (r[2][0] << 16);
    patch[5] = __funnelshift_r(r[2][0], r[2][1], 16);
    patch[6] = (r[2][1] >> 16) | (r[2][2] << 16);
  } else {
#pragma unroll
  for (int kh = 0; kh < KH; ++kh) {
    const int hi = hi0 + kh;
    const bool row_ok = hi >= 0 && hi < p.H;
#pragma unroll
    for (int kw = 0; kw < KW; ++kw) {
      const int wi = wi0 + kw;
      const bool ok = row_ok && wi >= 0 && wi < p.W;
      const uint8_t *ip = in_n + (static_cast<int64_t>(ok ? hi : 0) * p.W + (ok ? wi : 0)) * C;
#pragma unroll
      for (int c = 0; c < C; ++c) {
        const int d = (kh * KW + kw) * C + c;  // compile-time
        const uint32_t v = ok ? static_cast<uint32_t>(__ldg(ip + c)) : zi;
        patch[d >> 2] |= v << (8 * (d & 3));
      }
    }
  }
  }
  uint32_t sum_in = 0;
#pragma unroll
  for (int i = 0; i < DW; ++i) sum_in = __dp4a(patch[i], 0x01010101u, sum_in);
  const int32_t in_term = -p.zp_f * static_cast<int32_t>(sum_in);
  uint8_t *outp = p.out + pix * p.O;
  // The requantization variant is chosen once per thread, and output channels are handled four
  // at a time without per-channel checks when O is a multiple of four: in a loop this short a
  // branch per value costs more than the arithmetic.
  if ((p.O & 3) == 0) {
    switch (p.rq_variant) {
      case 5: patch_outputs<DW, DWP, 5>(patch, smem_w, cterm, in_term, p, outp); break;
      case 4: patch_outputs<DW, DWP, 4>(patch, smem_w, cterm, in_term, p, outp); break;
      case 3: patch_outputs<DW, DWP, 3>(patch, smem_w, cterm, in_term, p, outp); break;
      case 2: patch_outputs<DW, DWP, 2>(patch, smem_w, cterm, in_term, p, outp); break;
      case 1: patch_outputs<DW, DWP, 1>(patch, smem_w, cterm, in_term, p, outp); break;
      default: patch_outputs<DW, DWP, 0>(patch, smem_w, cterm, in_term, p, outp); break;
    }
    continue;
  }
  for (int o = 0; o < p.O; ++o) {
    const uint32_t *wr = smem_w + o * DWP;
    uint32_t dot = 0;
#pragma unroll
    for (int q = 0; q < DW; ++q) dot = __dp4a(patch[q], wr[q], dot);
    outp[o] = static_cast<uint8_t>(mb_requant_fast(static_cast<int32_t>(dot) + in_term + cterm[o], p.rq));
  }
  }
}

// Patch gather: row `pix` of the [pixels x depth_padded] matrix receives the
// KH*KW*C bytes under the filter window.  Out-of-image taps and the alignment
// tail beyond `depth` hold zp_in, so that they contribute
// (zp_in - zp_in) * (w - zp_f) = 0 whatever the filter side holds.
__global__ void __launch_bounds__(256) im2col_u8_kernel(const ConvParams p, uint8_t *col) {
  const int64_t npix = static_cast<int64_t>(p.N) * p.Ho * p.Wo;
  const int taps = p.KH * p.KW;
  // one thread per (pixel, tap): copies C bytes
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= npix * (taps + 1)) return;
  const int64_t pix = tid / (taps + 1);
  const int tap = static_cast<int>(tid % (taps + 1));
  uint8_t *dst = col + pix * p.depth_padded;
  if (tap == taps) {  // alignment tail
    for (int i = p.depth; i < p.depth_padded; ++i) dst[i] = static_cast<uint8_t>(p.zp_in);
    return;
  }
  const int kh = tap / p.KW, kw = tap % p.KW;
  const int wo = static_cast<int>(pix % p.Wo);
  const int ho = static_cast<int>((pix / p.Wo) % p.Ho);
  const int n = static_cast<int>(pix / (static_cast<int64_t>(p.Wo) * p.Ho));
  const int hi = ho * p.stride_h - p.pad_top + kh, wi = wo * p.stride_w - p.pad_left + kw;
  dst += tap * p.C;
  if (hi < 0 || hi >= p.H || wi < 0 || wi >= p.W) {
    const uint8_t padv = static_cast<uint8_t>(p.zp_in);
    for (int c = 0; c < p.C; ++c) dst[c] = padv;
  } else {
    const uint8_t *src = p.in + ((static_cast<int64_t>(n) * p.H + hi) * p.W + wi) * p.C;
    if ((p.C & 15) == 0 && (p.depth_padded & 15) == 0 &&
        ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0) {
      for (int c = 0; c < p.C; c += 16)
        *reinterpret_cast<uint4 *>(dst + c) = __ldg(reinterpret_cast<const uint4 *>(src + c));
    } else {
      for (int c = 0; c < p.C; ++c) dst[c] = src[c];
    }
  }
}

// Copy the [O x depth] filter into [O x depth_padded] with a zero tail.
__global__ void __launch_bounds__(256) pad_rows_u8_kernel(const uint8_t *__restrict__ src,
                                                          uint8_t *__restrict__ dst, int64_t rows,
                                                          int len, int len_padded) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= rows * len_padded) return;
  const int64_t r = tid / len_padded;
  const int i = static_cast<int>(tid % len_padded);
  dst[tid] = i < len ? src[r * len + i] : 0;
}

}  // namespace

extern "C" int mb_conv2d_u8_nhwc(mb_context *ctx, const uint8_t *in, const uint8_t *filter,
                                 const int32_t *bias, uint8_t *out, int64_t N, int64_t H,
                                 int64_t W, int64_t C, int64_t O, int64_t KH, int64_t KW,
                                 int stride_h, int stride_w, int pad_top, int pad_left,
                                 int64_t Ho, int64_t Wo, int32_t zp_in, int32_t zp_f,
                                 int32_t multiplier, int32_t right_shift, int32_t zp_out) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (N < 0 || H < 1 || W < 1 || C < 1 || O < 1 || KH < 1 || KW < 1 || Ho < 0 || Wo < 0 ||
      stride_h < 1 || stride_w < 1 || pad_top < 0 || pad_left < 0)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_conv2d_u8_nhwc: bad shape argument");
  if (N == 0 || Ho == 0 || Wo == 0) return MB_SUCCESS;
  if (in == nullptr || filter == nullptr || out == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_conv2d_u8_nhwc: null operand");
  if (multiplier <= 0 || right_shift < 0 || right_shift > 31)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_conv2d_u8_nhwc: bad multiplier/shift");
  if (zp_in < 0 || zp_in > 255 || zp_out < 0 || zp_out > 255)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_conv2d_u8_nhwc: zero point outside uint8");
  const int64_t depth = C * KH * KW;
  const int64_t pixels = N * Ho * Wo;
  if (depth > (1 << 24) || pixels >= (1ll << 31) || H > (1 << 20) || W > (1 << 20))
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_conv2d_u8_nhwc: tensor too large");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));

  if (KH == 1 && KW == 1 && stride_h == 1 && stride_w == 1 && pad_top == 0 && pad_left == 0 &&
      Ho == H && Wo == W) {
    // out[pixel][o] = sum_c in[pixel][c] * filter[o][c]: A = input (K-major),
    // B^T = filter (K-major), C row-major = NHWC, bias per column (= channel).
    return mb_gemm_u8_rowmajor(ctx, in, filter, bias, out, 0, 1, pixels, O, depth, false, false,
                               0, 0, zp_in, zp_f, multiplier, right_shift, zp_out, 0);
  }

  ConvParams p;
  p.in = in; p.filter = filter; p.bias = bias; p.out = out;
  p.N = static_cast<int>(N); p.H = static_cast<int>(H); p.W = static_cast<int>(W);
  p.C = static_cast<int>(C); p.O = static_cast<int>(O);
  p.KH = static_cast<int>(KH); p.KW = static_cast<int>(KW);
  p.stride_h = stride_h; p.stride_w = stride_w; p.pad_top = pad_top; p.pad_left = pad_left;
  p.Ho = static_cast<int>(Ho); p.Wo = static_cast<int>(Wo);
  p.depth = static_cast<int>(depth);
  p.depth_padded = static_cast<int>(align_up(static_cast<size_t>(depth), 16));
  p.zp_in = zp_in; p.zp_f = zp_f;
  p.rq = mb_make_requant(multiplier, right_shift, zp_out);
  p.rq_variant = mb_requant_variant(right_shift, zp_out);

  if (KH == 3 && KW == 3 && C == 3 && O <= 256 &&
      (reinterpret_cast<uintptr_t>(out) & 3u) == 0) {
    const size_t smem = static_cast<size_t>(O) * (8 * 4 + 4);
    const unsigned blocks = static_cast<unsigned>(ceil_div64(pixels, 128));
    const unsigned grid = std::min<unsigned>(blocks, static_cast<unsigned>(ctx->num_sms) * 16u);
    MB_CUDA(ctx, mb_launch_chained(ctx, conv_u8_patch_dp4a_kernel<3, 3, 3>, dim3(grid), dim3(128), smem, p));
    MB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
    return MB_SUCCESS;
  }
  const size_t direct_smem = static_cast<size_t>(depth) * O * sizeof(int16_t);
  if (direct_smem <= 32 * 1024 && depth <= 256) {
    const unsigned blocks = static_cast<unsigned>(ceil_div64(pixels, 128));
    if (O % 32 == 0 || O > 16) conv_u8_direct_kernel<32><<<blocks, 128, direct_smem, ctx->stream>>>(p);
    else conv_u8_direct_kernel<8><<<blocks, 128, direct_smem, ctx->stream>>>(p);
    MB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
    return MB_SUCCESS;
  }

  // Patch gather + GEMM.  The scratch block is carved here and by the GEMM;
  // the GEMM carves from the start of the arena, so the patch matrix and the
  // padded filter live in memory obtained separately for the duration of the
  // call.
  uint8_t *col = nullptr, *fpad = nullptr;
  const size_t col_bytes = static_cast<size_t>(pixels) * p.depth_padded;
  const bool pad_filter = p.depth_padded != p.depth;
  const size_t f_bytes = pad_filter ? static_cast<size_t>(O) * p.depth_padded : 0;
  MB_CUDA(ctx, cudaMallocAsync(reinterpret_cast<void **>(&col), col_bytes + f_bytes + 256, ctx->stream));
  fpad = col + align_up(col_bytes, 256);
  {
    const int64_t threads = pixels * (KH * KW + 1);
    im2col_u8_kernel<<<static_cast<unsigned>(ceil_div64(threads, 256)), 256, 0, ctx->stream>>>(p, col);
    ctx->launches++;
  }
  const uint8_t *f_use = filter;
  if (pad_filter) {
    const int64_t threads = O * p.depth_padded;
    pad_rows_u8_kernel<<<static_cast<unsigned>(ceil_div64(threads, 256)), 256, 0, ctx->stream>>>(
        filter, fpad, O, p.depth, p.depth_padded);
    ctx->launches++;
    f_use = fpad;
  }
  int st = mb_check_cuda(ctx, cudaGetLastError(), "im2col launch");
  if (st == MB_SUCCESS) {
    // The GEMM runs over depth_padded; the tail columns hold zp_in on the
    // patch side and therefore add nothing to the accumulator.
    st = mb_gemm_u8_rowmajor(ctx, col, f_use, bias, out, 0, 1, pixels, O, p.depth_padded, false,
                             false, 0, 0, zp_in, zp_f, multiplier, right_shift, zp_out, 0);
  }
  cudaFreeAsync(col, ctx->stream);
  return st;
}
