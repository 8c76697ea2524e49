// uint8 Conv2D, NHWC input, OHWI filter, NHWC output.
//
// Reference behaviour: Conv2dOp<RT_CPU,uint8_t>::Run (mace/ops/conv_2d.cc:
// 201-318): [im2col with the input zero point as pad value, :322-412] then a
// GEMM filter[O x depth] * patches[depth x pixels] with a per-output-channel
// int32 bias and the fixed-point output pipeline.  Padding with the zero point
// contributes (zp - zp) * w = 0, i.e. exactly the sum over in-bounds taps.
//
// Routes:
//   1x1 stride 1      -> the NHWC tensor already is the [pixels x C] K-major
//                        GEMM operand; no copy (conv_2d.cc:279-281); depth 32
//                        on many pixels: the thread-per-pixel kernel below
//   3x3 on 3 channels -> thread-per-pixel tensor-core kernel (namespace stem:
//                        MobileNet's 3x3x3 first layer), or the packed-patch
//                        dp4a kernel when the channel count is no multiple of 16
//   small depth * O   -> direct kernel, one thread per output pixel, the whole
//                        filter in shared memory
//   everything else   -> patch gather into scratch (rows padded to 16 bytes)
//                        + tensor-core GEMM
#include "common.cuh"
#include "sm100_ptx.cuh"

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
  // pixel index -> (image, row, column) without a hardware division: see FastDiv
  uint32_t wo_mul, wo_shift, ho_mul, ho_shift;
};

// Division of a dividend below 2^31 by a divisor fixed at launch: with s = ceil(log2 d) and
// m = ceil(2^(31 + s) / d) (which fits 32 bits), floor(n / d) = (n * m) >> (31 + s) for every
// n < 2^31, because m * d - 2^(31 + s) < d <= 2^s.  d = 1 is encoded as m = 0.
static inline void fast_div_make(uint32_t d, uint32_t *mul, uint32_t *shift) {
  if (d <= 1) { *mul = 0; *shift = 0; return; }
  uint32_t s = 0;
  while ((1ull << s) < d) ++s;
  *mul = static_cast<uint32_t>(((1ull << (31 + s)) + d - 1) / d);
  *shift = s - 1;
}
__device__ __forceinline__ uint32_t fast_div(uint32_t n, uint32_t mul, uint32_t shift) {
  return mul == 0 ? n : (__umulhi(n, mul) >> shift);
}

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

// The KH*KW*C bytes under the filter window of output pixel `pix`, packed into 32-bit words
// (byte d of the patch = tap (d / C) channel d % C; out-of-image taps hold the input zero point,
// the bytes past the patch are zero).
template <int KH, int KW, int C>
__device__ __forceinline__ void gather_patch(const ConvParams &p, int64_t pix, uint32_t (&patch)[(KH * KW * C + 3) / 4]) {
  constexpr int DEPTH = KH * KW * C;
  constexpr int DW = (DEPTH + 3) / 4;
  // (the pixel count is below 2^31: 32-bit divisions)
  const uint32_t pix32 = static_cast<uint32_t>(pix);
  const uint32_t row32 = fast_div(pix32, p.wo_mul, p.wo_shift);
  const int wo = static_cast<int>(pix32 - row32 * static_cast<uint32_t>(p.Wo));
  const int n = static_cast<int>(fast_div(row32, p.ho_mul, p.ho_shift));
  const int ho = static_cast<int>(row32 - static_cast<uint32_t>(n) * static_cast<uint32_t>(p.Ho));
  const int hi0 = ho * p.stride_h - p.pad_top, wi0 = wo * p.stride_w - p.pad_left;
  const uint8_t *in_n = p.in + static_cast<int64_t>(n) * p.H * p.W * C;
#pragma unroll
  for (int i = 0; i < DW; ++i) patch[i] = 0;
  const uint32_t zi = static_cast<uint32_t>(p.zp_in);
  // A row of a 3x3x3 window is 9 contiguous bytes (3 pixels x 3 channels).  Three aligned 32-bit
  // loads cover it, a funnel shift removes the misalignment, and the three rows are spliced into
  // the 27-byte patch at byte offsets 0, 9 and 18: 9 loads and about 50 logic instructions instead
  // of 27 byte loads with their address arithmetic and merges.  Taps outside the image take the
  // input zero point through byte masks (columns) and selects (rows), so border pixels follow the
  // same instruction stream as interior ones and a warp that holds a border pixel does not run
  // both versions.  The 12 bytes of a row's loads may start up to 3 bytes before and end up to
  // 3 bytes behind the 9 wanted ones: only pixels for which that would leave the tensor (its
  // first and last few bytes) take the byte-wise version below.
  bool words = false;
  if constexpr (KH == 3 && KW == 3 && C == 3) {
    // (the host sends only images of fewer than 2^31 bytes here: offsets inside an image are 32-bit)
    const int32_t img_bytes = p.H * p.W * 3;
    const uint32_t img_mis = static_cast<uint32_t>(n) * static_cast<uint32_t>(img_bytes);  // low bits decide the alignment
    const bool c0 = static_cast<unsigned>(wi0) < static_cast<unsigned>(p.W);
    const bool c1 = static_cast<unsigned>(wi0 + 1) < static_cast<unsigned>(p.W);
    const bool c2 = static_cast<unsigned>(wi0 + 2) < static_cast<unsigned>(p.W);
    int32_t first[3];   // offset, inside the image, of the aligned word that holds the row's first byte
    uint32_t sh[3];
    bool row_ok[3];
    words = (reinterpret_cast<uintptr_t>(p.in) & 3u) == 0;
#pragma unroll
    for (int kh = 0; kh < 3; ++kh) {
      const int hi = hi0 + kh;
      row_ok[kh] = static_cast<unsigned>(hi) < static_cast<unsigned>(p.H);
      const int32_t off = ((row_ok[kh] ? hi : 0) * p.W + wi0) * 3;
      const uint32_t mis = (img_mis + static_cast<uint32_t>(off)) & 3u;
      first[kh] = off - static_cast<int32_t>(mis);
      sh[kh] = mis * 8;
      words = words && (first[kh] >= 0 || n > 0) && (first[kh] + 12 <= img_bytes || n + 1 < p.N);
    }
    if (words) {
      const uint32_t zi4 = zi * 0x01010101u;
      const uint32_t m0 = (c0 ? 0x00ffffffu : 0u) | (c1 ? 0xff000000u : 0u);
      const uint32_t m1 = (c1 ? 0x0000ffffu : 0u) | (c2 ? 0xffff0000u : 0u);
      const uint32_t m2 = c2 ? 0xffu : 0u;
      uint32_t r[3][3];
#pragma unroll
      for (int kh = 0; kh < 3; ++kh) {
        const uint32_t *wp = reinterpret_cast<const uint32_t *>(in_n + first[kh]);
        const uint32_t w0 = __ldg(wp), w1 = __ldg(wp + 1), w2 = __ldg(wp + 2);
        const uint32_t f0 = __funnelshift_r(w0, w1, sh[kh]), f1 = __funnelshift_r(w1, w2, sh[kh]), f2 = w2 >> sh[kh];
        r[kh][0] = row_ok[kh] ? ((f0 & m0) | (zi4 & ~m0)) : zi4;
        r[kh][1] = row_ok[kh] ? ((f1 & m1) | (zi4 & ~m1)) : zi4;
        r[kh][2] = row_ok[kh] ? ((f2 & m2) | (zi & ~m2)) : zi;  // the row's ninth byte
      }
      patch[0] = r[0][0];
      patch[1] = r[0][1];
      patch[2] = r[0][2] | (r[1][0] << 8);
      patch[3] = __funnelshift_r(r[1][0], r[1][1], 24);
      patch[4] = (r[1][1] >> 24) | (r[1][2] << 8) | (r[2][0] << 16);
      patch[5] = __funnelshift_r(r[2][0], r[2][1], 16);
      patch[6] = (r[2][1] >> 16) | (r[2][2] << 16);
    }
  }
  if (!words) {
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
  uint32_t patch[DW];
  gather_patch<KH, KW, C>(p, pix, patch);
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

// ---- the same first-layer convolution with the products on the tensor core -----------------
// out[pixel][o] = sum_d patch[pixel][d] * filter[o][d] is a GEMM with K = 27: one tcgen05.mma
// (kind::i8, K = 32) per 128 pixels does what 7 dp4a per output value do above.  The block keeps
// the shape of the dp4a kernel -- 128 threads, a thread per pixel, several blocks per SM, whose
// latencies hide one another -- and per group of 128 pixels: every thread gathers its 27-byte
// patch (gather_patch) and stores it as a row of the MMA's A operand (K-major without swizzle:
// two planes of 16-byte pieces, [half of K][pixel][16 bytes]); one thread issues the MMA against
// B = the raw filter rows; every thread reads its pixel's row of the accumulator from tensor
// memory and applies
//   sum (in - zi)(f - zf) = sum in*f - zf * sum in + (bias - zi * sum f + depth * zi * zf)
// (the byte sum of its own patch: seven dp4a) and the requantization.  Each block holds as many
// columns of tensor memory as there are output channels (32 at least); registers let eight blocks
// share an SM, and the shared-memory request is padded so that never more blocks are resident
// than the SM's 512 columns serve.
namespace stem {

using namespace sm100;

struct Params {
  ConvParams c;
  int n_cols;     // MMA N = O (a multiple of 16)
  int acc_cols;   // tensor-memory columns of the block (power of two >= n_cols, at least 32)
  int64_t tiles;  // groups of 128 pixels
  int *status;
  int filter_const;  // filter and bias are not written by work enqueued ahead (weights): read them before the wait
};

// KD: 27 = the 3x3x3 window (gathered, zero tail up to 32); 32 / 64 / 128 = a pointwise layer
// of that depth, whose A row is the pixel's own KD contiguous bytes.
// GROUPS: the number of 16-channel groups when it is fixed at compile time (2, 4: the epilogue is
// then straight-line code without per-group address arithmetic), 0 = taken from the parameters.
template <int VAR, int KD, int GROUPS>
__global__ void __launch_bounds__(128, 8) conv_u8_stem_mma_kernel(const Params q) {
  constexpr int KPAD = KD == 27 ? 32 : KD;   // bytes of an A / B row
  constexpr int PLANES = KPAD / 16;          // 16-byte pieces per row
  const ConvParams &p = q.c;
  extern __shared__ uint8_t stem_raw[];
  const uint32_t base = (smem_u32(stem_raw) + 127u) & ~127u;
  uint8_t *sm = stem_raw + (base - smem_u32(stem_raw));
  // layout: A tile ([PLANES][128][16]) | B ([PLANES][n_cols][16]) | constants [O] | mbarrier, tmem slot
  uint8_t *b_tile = sm + PLANES * 2048;
  int32_t *cterm = reinterpret_cast<int32_t *>(b_tile + q.n_cols * KPAD);
  uint64_t *bar = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(cterm) + ((p.O * 4 + 127) & ~127));
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);
  const uint32_t mma_bar = smem_u32(bar);
  const int warp = threadIdx.x >> 5;
  mb_grid_dep_launch();
  if (threadIdx.x == 0) {
    mbar_init(mma_bar, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), static_cast<uint32_t>(q.acc_cols));
    tmem_relinquish();
  }
  if (!q.filter_const) mb_grid_dep_wait();
  // B: row o = the filter row (KD bytes, zero tail); byte k of row n lives at [k / 16][n][k % 16].
  const bool filter_words = KD != 27 && (reinterpret_cast<uintptr_t>(p.filter) & 15u) == 0;
  for (int i = threadIdx.x; i < q.n_cols * PLANES; i += 128) {
    const int n = i / PLANES, piece = i % PLANES;
    uint4 v4;
    if (filter_words) {
      v4 = __ldg(reinterpret_cast<const uint4 *>(p.filter + n * KD + piece * 16));
    } else {
      uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
      for (int b = 0; b < 16; ++b) {
        const int k = piece * 16 + b;
        uint32_t v = 0;
        if (k < KD) v = static_cast<uint32_t>(__ldg(p.filter + n * KD + k));
        w[b >> 2] |= v << (8 * (b & 3));
      }
      v4 = make_uint4(w[0], w[1], w[2], w[3]);
    }
    *reinterpret_cast<uint4 *>(b_tile + piece * q.n_cols * 16 + n * 16) = v4;
  }
  __syncthreads();
  for (int o = threadIdx.x; o < p.O; o += 128) {  // (from the tile just written: 16 bytes a load)
    uint32_t fs = 0;
#pragma unroll
    for (int piece = 0; piece < PLANES; ++piece) {
      const uint4 v = *reinterpret_cast<const uint4 *>(b_tile + piece * q.n_cols * 16 + o * 16);
      fs = __dp4a(v.x, 0x01010101u, fs);
      fs = __dp4a(v.y, 0x01010101u, fs);
      fs = __dp4a(v.z, 0x01010101u, fs);
      fs = __dp4a(v.w, 0x01010101u, fs);
    }
    cterm[o] = (p.bias != nullptr ? p.bias[o] : 0) - p.zp_in * static_cast<int32_t>(fs) + KD * p.zp_in * p.zp_f;
  }
  fence_proxy_async();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (q.filter_const) mb_grid_dep_wait();  // the pixels come from the kernel in front
  const uint32_t tmem_base = *tmem_slot;
  const int64_t npix = static_cast<int64_t>(p.N) * p.Ho * p.Wo;
  const uint32_t idesc = make_idesc(/*c s32*/ 2, /*a u8*/ 0, /*b u8*/ 0, false, false, 128, static_cast<uint32_t>(q.n_cols));
  // K-major without swizzle: 8-row x 16-byte core matrices, 128 bytes from one group of 8 rows to
  // the next, a plane (all rows) from one 16-byte piece of K to the next; an MMA covers two planes
  const uint64_t a_desc = make_smem_desc(base, 2048, 128, 0);
  const uint64_t b_desc = make_smem_desc(smem_u32(b_tile), static_cast<uint32_t>(q.n_cols) * 16, 128, 0);
  const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  const int groups = GROUPS != 0 ? GROUPS : (p.O >> 4);
  const int n_out = GROUPS != 0 ? GROUPS * 16 : p.O;
  __shared__ int give_up;
  if (threadIdx.x == 0) give_up = 0;
  uint32_t phase = 0;
  for (int64_t t = blockIdx.x; t < q.tiles; t += gridDim.x, phase ^= 1) {
    const int64_t pix = t * 128 + threadIdx.x;
    uint32_t sum_in = 0;
    if constexpr (KD == 27) {
      uint32_t patch[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (pix < npix) gather_patch<3, 3, 3>(p, pix, reinterpret_cast<uint32_t (&)[7]>(patch));
#pragma unroll
      for (int i = 0; i < 7; ++i) sum_in = __dp4a(patch[i], 0x01010101u, sum_in);
      *reinterpret_cast<uint4 *>(sm + threadIdx.x * 16) = make_uint4(patch[0], patch[1], patch[2], patch[3]);
      *reinterpret_cast<uint4 *>(sm + 2048 + threadIdx.x * 16) = make_uint4(patch[4], patch[5], patch[6], 0);
    } else {
      // the pixel's own row, four 16-byte pieces at a time (all four requested before the first is used)
      const uint4 *row = reinterpret_cast<const uint4 *>(p.in + pix * KD);
#pragma unroll
      for (int p0 = 0; p0 < PLANES; p0 += 4) {
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (p0 + j < PLANES) v[j] = pix < npix ? __ldg(row + p0 + j) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (p0 + j < PLANES) {
            sum_in = __dp4a(v[j].x, 0x01010101u, sum_in);
            sum_in = __dp4a(v[j].y, 0x01010101u, sum_in);
            sum_in = __dp4a(v[j].z, 0x01010101u, sum_in);
            sum_in = __dp4a(v[j].w, 0x01010101u, sum_in);
            *reinterpret_cast<uint4 *>(sm + (p0 + j) * 2048 + threadIdx.x * 16) = v[j];
          }
      }
    }
    fence_proxy_async();
    tc_fence_before_sync();
    __syncthreads();  // the tile is complete; every warp has read the previous accumulator
    if (threadIdx.x == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int kk = 0; kk < PLANES / 2; ++kk)
        mma_i8_ss(tmem_base, a_desc + static_cast<uint64_t>(kk * (4096 >> 4)),
                  b_desc + static_cast<uint64_t>(kk * ((q.n_cols * 32) >> 4)), idesc, kk > 0 ? 1u : 0u);
      mma_commit(mma_bar);
      // one thread waits for the MMA (bounded; on a timeout the block records it and leaves), the
      // others wait at the block barrier, which costs no issue slots
      bool done = mbar_try_wait(mma_bar, phase);
      if (!done) {
        const long long start = clock64();
        while (!(done = mbar_try_wait(mma_bar, phase))) {
          __nanosleep(32);
          if (clock64() - start > (1ll << 31)) break;
        }
      }
      if (!done) give_up = 1;
    }
    __syncthreads();
    if (give_up != 0) {
      if (threadIdx.x == 0) atomicCAS(q.status, 0, MB_DEV_TIMEOUT_MMA);
      break;
    }
    tc_fence_after_sync();
    const int32_t in_term = -p.zp_f * static_cast<int32_t>(sum_in);
    auto emit = [&](const uint32_t (&v)[16], int cg) {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int4 ct = *reinterpret_cast<const int4 *>(cterm + cg * 16 + 4 * j);
        const int32_t a0 = static_cast<int32_t>(v[4 * j + 0]) + in_term + ct.x;
        const int32_t a1 = static_cast<int32_t>(v[4 * j + 1]) + in_term + ct.y;
        const int32_t a2 = static_cast<int32_t>(v[4 * j + 2]) + in_term + ct.z;
        const int32_t a3 = static_cast<int32_t>(v[4 * j + 3]) + in_term + ct.w;
        if (VAR >= 4) {
          w[j] = mb_requant_pack4<VAR == 5>(a0, a1, a2, a3, p.rq);
        } else {
          w[j] = mb_requant_fast(a0, p.rq) | (mb_requant_fast(a1, p.rq) << 8) | (mb_requant_fast(a2, p.rq) << 16) |
                 (mb_requant_fast(a3, p.rq) << 24);
        }
      }
      if (pix < npix) *reinterpret_cast<uint4 *>(p.out + pix * n_out + cg * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    };
    // two groups of 16 channels per round trip to tensor memory
#pragma unroll
    for (int cg = 0; cg < groups; cg += 2) {
      uint32_t v0[16], v1[16];
      const bool two = cg + 1 < groups;
      tmem_ld_32x32b_x16(taddr + cg * 16, v0);
      if (two) tmem_ld_32x32b_x16(taddr + (cg + 1) * 16, v1);
      tmem_ld_wait_x16(v0);
      emit(v0, cg);
      if (two) {
        tmem_ld_wait_x16(v1);
        emit(v1, cg + 1);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(q.acc_cols));
  }
}

template <int KD, int GROUPS>
static int launch_kdg(mb_context *ctx, const Params &q, unsigned grid, size_t smem, int attr_bit) {
  const int var = q.c.rq_variant == 5 ? 5 : q.c.rq_variant == 4 ? 4 : 0;
  if (!(ctx->func_attr_mask2 & (1ull << attr_bit))) {
    MB_CUDA(ctx, cudaFuncSetAttribute(conv_u8_stem_mma_kernel<5, KD, GROUPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024));
    MB_CUDA(ctx, cudaFuncSetAttribute(conv_u8_stem_mma_kernel<4, KD, GROUPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024));
    MB_CUDA(ctx, cudaFuncSetAttribute(conv_u8_stem_mma_kernel<0, KD, GROUPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024));
    ctx->func_attr_mask2 |= (1ull << attr_bit);
  }
  if (var == 5) MB_CUDA(ctx, mb_launch_chained(ctx, conv_u8_stem_mma_kernel<5, KD, GROUPS>, dim3(grid), dim3(128), smem, q));
  else if (var == 4) MB_CUDA(ctx, mb_launch_chained(ctx, conv_u8_stem_mma_kernel<4, KD, GROUPS>, dim3(grid), dim3(128), smem, q));
  else MB_CUDA(ctx, mb_launch_chained(ctx, conv_u8_stem_mma_kernel<0, KD, GROUPS>, dim3(grid), dim3(128), smem, q));
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

template <int KD>
static int launch_kd(mb_context *ctx, const Params &q, unsigned grid, size_t smem, int attr_bit) {
  if (KD <= 32 && q.n_cols == 32) return launch_kdg<KD, (KD <= 32 ? 2 : 0)>(ctx, q, grid, smem, attr_bit + 1);
  if (KD <= 32 && q.n_cols == 64) return launch_kdg<KD, (KD <= 32 ? 4 : 0)>(ctx, q, grid, smem, attr_bit + 2);
  return launch_kdg<KD, 0>(ctx, q, grid, smem, attr_bit);
}

// kd: 27 (the 3x3x3 window) or the depth of a pointwise layer (32, 64, 128); O a multiple of 16, at
// most 256; the output 16-byte aligned (and the input too, for a pointwise layer).
static int launch(mb_context *ctx, const ConvParams &p, int kd, int64_t pixels) {
  Params q;
  q.c = p;
  q.n_cols = p.O;
  q.acc_cols = q.n_cols <= 32 ? 32 : q.n_cols <= 64 ? 64 : q.n_cols <= 128 ? 128 : 256;
  q.tiles = ceil_div64(pixels, 128);
  q.status = ctx->dev_status;
  q.filter_const = ctx->conv_filter_const;
  const int kpad = kd == 27 ? 32 : kd;
  const int per_sm = 512 / q.acc_cols;
  // (the request is padded so that no more blocks fit an SM than its tensor memory serves: a
  // further block would sit in tcgen05.alloc until another one has finished all its pixels)
  const size_t smem = std::max<size_t>(128 + static_cast<size_t>(kpad / 16) * 2048 + static_cast<size_t>(q.n_cols) * kpad +
                                           align_up(static_cast<size_t>(p.O) * 4, 128) + 64,
                                       static_cast<size_t>(208 * 1024) / per_sm);
  // blocks: registers let eight be resident per SM; stem_grid = 1 launches exactly those, 2 twice as many
  const int resident = std::min(per_sm, 8);
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>(q.tiles, static_cast<int64_t>(ctx->num_sms) * resident * ctx->stem_grid));
  switch (kd) {
    case 27: return launch_kd<27>(ctx, q, grid, smem, 0);
    case 32: return launch_kd<32>(ctx, q, grid, smem, 3);
    case 64: return launch_kd<64>(ctx, q, grid, smem, 6);
    default: return launch_kd<128>(ctx, q, grid, smem, 9);
  }
}

}  // namespace stem

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
    // a short depth makes a 128-pixel tile of the persistent GEMM mostly hand-over: such layers
    // take the thread-per-pixel kernel (see namespace stem)
    if (ctx->thin_pw && ctx->use_tensor_cores && (C == 32 || (C == 64 && ctx->thin_pw >= 2) || (C == 128 && ctx->thin_pw >= 3)) && O % 16 == 0 &&
        O <= 128 && pixels >= 128 * static_cast<int64_t>(ctx->num_sms) &&
        ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(in)) & 15u) == 0) {
      ConvParams p;
      p.in = in; p.filter = filter; p.bias = bias; p.out = out;
      p.N = static_cast<int>(N); p.H = static_cast<int>(H); p.W = static_cast<int>(W);
      p.C = static_cast<int>(C); p.O = static_cast<int>(O);
      p.KH = 1; p.KW = 1; p.stride_h = 1; p.stride_w = 1; p.pad_top = 0; p.pad_left = 0;
      p.Ho = static_cast<int>(Ho); p.Wo = static_cast<int>(Wo);
      p.depth = static_cast<int>(depth); p.depth_padded = p.depth;
      p.zp_in = zp_in; p.zp_f = zp_f;
      p.rq = mb_make_requant(multiplier, right_shift, zp_out);
      p.rq_variant = mb_requant_variant(right_shift, zp_out);
      p.wo_mul = p.wo_shift = p.ho_mul = p.ho_shift = 0;
      return stem::launch(ctx, p, static_cast<int>(C), pixels);
    }
    ctx->gemm_b_const = ctx->conv_filter_const;  // the filter is the GEMM's B
    const int st = mb_gemm_u8_rowmajor(ctx, in, filter, bias, out, 0, 1, pixels, O, depth, false, false,
                                       0, 0, zp_in, zp_f, multiplier, right_shift, zp_out, 0);
    ctx->gemm_b_const = 0;
    return st;
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
  fast_div_make(static_cast<uint32_t>(Wo), &p.wo_mul, &p.wo_shift);
  fast_div_make(static_cast<uint32_t>(Ho), &p.ho_mul, &p.ho_shift);
  const bool image_32bit = H * W * C < (1ll << 31) - 16;

  if (image_32bit && ctx->stem_tc && ctx->use_tensor_cores && KH == 3 && KW == 3 && C == 3 && O % 16 == 0 && O <= 256 &&
      (reinterpret_cast<uintptr_t>(out) & 15u) == 0 && pixels >= 128)
    return stem::launch(ctx, p, 27, pixels);
  if (image_32bit && KH == 3 && KW == 3 && C == 3 && O <= 256 &&
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
