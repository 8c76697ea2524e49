// fp32 kernels of the path: batched GEMM, GEMV, general direct Conv2D and
// depthwise conv in NCHW, with bias and activation fused into the epilogue.
//
// Reference behaviour: ref::Gemm / ref::Gemv / ref::Conv2d / ref::DepthwiseConv2d
// (mace/ops/ref/gemm.cc:57-106, gemv.cc:45-81, conv_2d.cc:36-122,
// depthwise_conv_2d.cc:36-125), ref::BiasAdd (bias_add.cc:74-103) and
// ref::Activation (activation.cc:61-88).  The reference accumulates in fp32 in
// index order; these kernels accumulate in fp32 in a tiled order, so results
// agree to rounding (tests bound the difference at 1e-4 of the output range).
#include "common.cuh"

bool mb_gemm_f32_tc_supported(const mb_context *ctx, const float *X, const float *W, int64_t Mdim,
                              int64_t Ndim, int64_t K, int64_t x_row_stride, int64_t x_batch_stride,
                              int64_t w_row_stride, int64_t w_batch_stride);
int mb_gemm_f32_tc_launch(mb_context *ctx, const float *X, const float *W, const float *bias, float *C,
                          int64_t batch, int64_t Mdim, int64_t Ndim, int64_t K, int64_t x_row_stride,
                          int64_t x_batch_stride, int64_t w_row_stride, int64_t w_batch_stride,
                          int64_t c_row_stride, int64_t c_batch_stride, int act, float max_limit,
                          float coef, const float *residual);

namespace {

// ---- GEMM: 64 x 64 tile per 256-thread block, 4 x 4 outputs per thread ----------
constexpr int FT = 64;
constexpr int FK = 16;

struct GemmF32Params {
  const float *A, *B;
  float *C;
  const float *bias;  // per row of C (output channel) or null
  int64_t M, N, K;
  int64_t a_rs, a_cs, b_rs, b_cs, c_rs, c_cs;  // element strides
  int64_t a_bs, b_bs, c_bs;                    // batch strides
  int act;
  float max_limit, coef;
};

__global__ void __launch_bounds__(256) gemm_f32_kernel(const GemmF32Params p) {
  __shared__ float As[FK][FT + 4];
  __shared__ float Bs[FK][FT + 4];
  const int b = blockIdx.z;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * FT, n0 = static_cast<int64_t>(blockIdx.x) * FT;
  const float *A = p.A + b * p.a_bs, *B = p.B + b * p.b_bs;
  float *C = p.C + b * p.c_bs;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < p.K; k0 += FK) {
    for (int i = threadIdx.x; i < FK * FT; i += 256) {
      int kk, mm;
      if (p.a_cs == 1) { kk = i % FK; mm = i / FK; } else { mm = i % FT; kk = i / FT; }
      const int64_t m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < p.M && k < p.K) ? __ldg(A + m * p.a_rs + k * p.a_cs) : 0.f;
      int nn;
      if (p.b_cs == 1) { nn = i % FT; kk = i / FT; } else { kk = i % FK; nn = i / FK; }
      const int64_t n = n0 + nn, kb = k0 + kk;
      Bs[kk][nn] = (n < p.N && kb < p.K) ? __ldg(B + kb * p.b_rs + n * p.b_cs) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < FK; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
    const float bv = p.bias != nullptr ? p.bias[m] : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      float v = acc[i][j];
      if (p.bias != nullptr) v += bv;
      C[m * p.c_rs + n * p.c_cs] = mb_activate(v, p.act, p.max_limit, p.coef);
    }
  }
}

// ---- GEMV: one warp per matrix row ------------------------------------------------
__global__ void __launch_bounds__(256)
gemv_f32_kernel(const float *__restrict__ lhs, const float *__restrict__ rhs,
                const float *__restrict__ bias, float *__restrict__ out, int64_t batch,
                int64_t rows, int64_t K, int lhs_batched, int rhs_batched, int batch_chunk) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t b0 = static_cast<int64_t>(blockIdx.y) * batch_chunk;
  const int64_t b1 = min(batch, b0 + batch_chunk);
  for (int64_t b = b0; b < b1; ++b) {
    const float *lp = lhs + (lhs_batched ? b * rows * K : 0) + row * K;
    const float *rp = rhs + (rhs_batched ? b * K : 0);
    float s = 0.f;
    for (int64_t i = lane; i < K; i += 32) s = fmaf(__ldg(lp + i), __ldg(rp + i), s);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[b * rows + row] = s + (bias != nullptr ? bias[row] : 0.f);
  }
}

// ---- direct convolutions ------------------------------------------------------------
struct ConvF32Params {
  const float *in, *filter, *bias;
  float *out;
  int N, C, H, W, O, KH, KW, sh, sw, dh, dw, pad_t, pad_l, Ho, Wo, mult_ch;
  int act;
  float max_limit, coef;
};

// One thread per output value; the loop order (c, kh, kw) is the reference's.
__global__ void __launch_bounds__(256) conv2d_f32_direct_kernel(const ConvF32Params p) {
  const int64_t total = static_cast<int64_t>(p.N) * p.O * p.Ho * p.Wo;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int w = static_cast<int>(tid % p.Wo);
  int64_t r = tid / p.Wo;
  const int h = static_cast<int>(r % p.Ho);
  r /= p.Ho;
  const int m = static_cast<int>(r % p.O);
  const int n = static_cast<int>(r / p.O);
  float sum = 0.f;
  for (int c = 0; c < p.C; ++c) {
    const float *ib = p.in + (static_cast<int64_t>(n) * p.C + c) * p.H * p.W;
    const float *fp = p.filter + (static_cast<int64_t>(m) * p.C + c) * p.KH * p.KW;
    for (int kh = 0; kh < p.KH; ++kh) {
      const int ih = -p.pad_t + h * p.sh + kh * p.dh;
      if (ih < 0 || ih >= p.H) continue;
      for (int kw = 0; kw < p.KW; ++kw) {
        const int iw = -p.pad_l + w * p.sw + kw * p.dw;
        if (iw < 0 || iw >= p.W) continue;
        sum = fmaf(__ldg(ib + ih * p.W + iw), __ldg(fp + kh * p.KW + kw), sum);
      }
    }
  }
  if (p.bias != nullptr) sum += p.bias[m];
  p.out[tid] = mb_activate(sum, p.act, p.max_limit, p.coef);
}

__global__ void __launch_bounds__(256) dwconv_f32_kernel(const ConvF32Params p) {
  const int OC = p.C * p.mult_ch;
  const int64_t total = static_cast<int64_t>(p.N) * OC * p.Ho * p.Wo;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int w = static_cast<int>(tid % p.Wo);
  int64_t r = tid / p.Wo;
  const int h = static_cast<int>(r % p.Ho);
  r /= p.Ho;
  const int m = static_cast<int>(r % OC);
  const int n = static_cast<int>(r / OC);
  const int c = m / p.mult_ch, o = m % p.mult_ch;
  const float *ib = p.in + (static_cast<int64_t>(n) * p.C + c) * p.H * p.W;
  const float *fp = p.filter + (static_cast<int64_t>(o) * p.C + c) * p.KH * p.KW;
  float sum = 0.f;
  for (int kh = 0; kh < p.KH; ++kh) {
    const int ih = -p.pad_t + h * p.sh + kh * p.dh;
    if (ih < 0 || ih >= p.H) continue;
    for (int kw = 0; kw < p.KW; ++kw) {
      const int iw = -p.pad_l + w * p.sw + kw * p.dw;
      if (iw < 0 || iw >= p.W) continue;
      sum = fmaf(__ldg(ib + ih * p.W + iw), __ldg(fp + kh * p.KW + kw), sum);
    }
  }
  if (p.bias != nullptr) sum += p.bias[m];
  p.out[tid] = mb_activate(sum, p.act, p.max_limit, p.coef);
}

// ---- im2col for the tensor-core route of the general convolution --------------------------
// col[k][...] with k = (c * KH + kh) * KW + kw, the order of an OIHW filter row.  Two layouts:
// per image (col_ns = K * col_rs: image n owns a [K x positions] matrix) and merged
// (col_ns = positions per image: the images of a chunk lie side by side in one
// [K x images * positions] matrix, which keeps 128-position tiles full when an image has few).
struct ColF32Params {
  const float *in;  // first image of the chunk
  float *col;
  int C, H, W, KH, KW, sh, sw, dh, dw, pad_t, pad_l, Ho, Wo, hw;
  int64_t col_rs, col_ns;
};

// One block per (group of output rows, channel and filter row, image): threadIdx.x walks along
// an output row and threadIdx.y picks the row, so no thread divides by anything, the KW taps
// of a pixel re-read the same input row from L1, and every store is a contiguous run.
__global__ void __launch_bounds__(128) im2col_f32_kernel(const ColF32Params p, int rows_per_block) {
  const int h = blockIdx.x * blockDim.y + threadIdx.y, n = blockIdx.z;
  if (h >= p.Ho) return;
  const float *__restrict__ in = p.in;
  float *__restrict__ col = p.col;
  const int y_end = min((static_cast<int>(blockIdx.y) + 1) * rows_per_block, p.C * p.KH);
  // Up to eight values are loaded before the first is stored: a store waits for the load that
  // feeds it, a warp issues in order, and the compiler may not move a load above a store to
  // memory it cannot tell apart.
  if (p.KW == 1) {
    for (int w = threadIdx.x; w < p.Wo; w += blockDim.x) {
      const int iw = w * p.sw - p.pad_l;
      const bool col_ok = iw >= 0 && iw < p.W;
      for (int y0 = blockIdx.y * rows_per_block; y0 < y_end; y0 += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int y = y0 + j;
          const int c = y / p.KH, kh = y - c * p.KH;
          const int ih = h * p.sh - p.pad_t + kh * p.dh;
          const bool ok = y < y_end && col_ok && ih >= 0 && ih < p.H;
          v[j] = ok ? __ldg(in + ((static_cast<int64_t>(n) * p.C + c) * p.H + ih) * p.W + iw) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (y0 + j < y_end) col[static_cast<int64_t>(y0 + j) * p.col_rs + n * p.col_ns + h * p.Wo + w] = v[j];
      }
    }
    return;
  }
  for (int y = blockIdx.y * rows_per_block; y < y_end; ++y) {  // y = c * KH + kh
    const int c = y / p.KH, kh = y - c * p.KH;
    const int ih = h * p.sh - p.pad_t + kh * p.dh;
    const bool row_ok = ih >= 0 && ih < p.H;
    const float *src = in + ((static_cast<int64_t>(n) * p.C + c) * p.H + (row_ok ? ih : 0)) * p.W;
    float *dst = col + static_cast<int64_t>(y) * p.KW * p.col_rs + n * p.col_ns + h * p.Wo;
    for (int w = threadIdx.x; w < p.Wo; w += blockDim.x) {
      const int iw0 = w * p.sw - p.pad_l;
      for (int kw0 = 0; kw0 < p.KW; kw0 += 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int iw = iw0 + (kw0 + j) * p.dw;
          v[j] = (kw0 + j < p.KW && row_ok && iw >= 0 && iw < p.W) ? __ldg(src + iw) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (kw0 + j < p.KW) dst[(kw0 + j) * p.col_rs + w] = v[j];
      }
    }
  }
}

// rows of K floats -> rows of Kp floats (a 16-byte multiple, which a tensor map's strides need)
__global__ void __launch_bounds__(256)
repack_rows_f32_kernel(const float *__restrict__ src, float *__restrict__ dst, int64_t rows, int K, int Kp) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= rows * Kp) return;
  const int k = static_cast<int>(i % Kp);
  dst[i] = k < K ? __ldg(src + (i / Kp) * K + k) : 0.f;
}

// merged product [O][images * hw] (row stride src_rs) -> NCHW images
__global__ void __launch_bounds__(256)
unmerge_f32_kernel(const float *__restrict__ src, float *__restrict__ dst, int64_t total, int O, int hw,
                   int64_t src_rs) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= total) return;
  const int pos = static_cast<int>(i % hw);
  const int64_t r = i / hw;
  const int o = static_cast<int>(r % O);
  const int64_t n = r / O;
  dst[i] = __ldg(src + o * src_rs + n * hw + pos);
}

// out[c][r] = in[r][c] for a [rows x cols] matrix, through a 32 x 33 shared-memory tile.
__global__ void __launch_bounds__(256)
transpose_f32_kernel(const float *__restrict__ in, float *__restrict__ out, int rows, int cols) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8)
    if (r0 + i < rows && c0 + tx < cols) tile[i][tx] = __ldg(in + static_cast<int64_t>(r0 + i) * cols + c0 + tx);
  __syncthreads();
  for (int i = ty; i < 32; i += 8)
    if (c0 + i < cols && r0 + tx < rows) out[static_cast<int64_t>(c0 + i) * rows + r0 + tx] = tile[tx][i];
}

}  // namespace

// Strided batched fp32 GEMM with optional per-row bias and activation; the
// building block of the 1x1 convolution and of the Winograd batched product.
int mb_gemm_f32_strided(mb_context *ctx, const float *A, const float *B, float *C,
                        const float *bias_per_row, int64_t batch, int64_t M, int64_t N, int64_t K,
                        int64_t a_rs, int64_t a_cs, int64_t a_bs, int64_t b_rs, int64_t b_cs,
                        int64_t b_bs, int64_t c_rs, int64_t c_cs, int64_t c_bs, int act,
                        float max_limit, float coef) {
  // C = A * B with A [M x K] k-contiguous, B [K x N] n-contiguous and C n-contiguous is the
  // tensor-core kernel's layout with the roles X = B (pixels x channels side), W = A.
  if (a_cs == 1 && b_cs == 1 && c_cs == 1 &&
      mb_gemm_f32_tc_supported(ctx, B, A, N, M, K, b_rs, b_bs, a_rs, a_bs)) {
    return mb_gemm_f32_tc_launch(ctx, B, A, bias_per_row, C, batch, N, M, K, b_rs, b_bs, a_rs, a_bs,
                                 c_rs, c_bs, act, max_limit, coef, nullptr);
  }
  if (batch > 65535 || ceil_div64(M, FT) > 65535)
    return mb_fail(ctx, MB_UNSUPPORTED, "fp32 GEMM: batch or M too large for this kernel");
  GemmF32Params p;
  p.A = A; p.B = B; p.C = C; p.bias = bias_per_row;
  p.M = M; p.N = N; p.K = K;
  p.a_rs = a_rs; p.a_cs = a_cs; p.b_rs = b_rs; p.b_cs = b_cs; p.c_rs = c_rs; p.c_cs = c_cs;
  p.a_bs = a_bs; p.b_bs = b_bs; p.c_bs = c_bs;
  p.act = act; p.max_limit = max_limit; p.coef = coef;
  dim3 grid(static_cast<unsigned>(ceil_div64(N, FT)), static_cast<unsigned>(ceil_div64(M, FT)),
            static_cast<unsigned>(batch));
  gemm_f32_kernel<<<grid, 256, 0, ctx->stream>>>(p);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

// General convolution as im2col + GEMM (the tensor-core kernel when the shapes allow it).
// Images are processed in chunks so that the column matrix stays below the context's budget
// (1 GiB unless the option col_budget_mb changes it).
static int conv2d_f32_im2col(mb_context *ctx, const float *in, const float *filter, const float *bias,
                             float *out, int64_t N, int64_t C, int64_t H, int64_t W, int64_t O,
                             int64_t KH, int64_t KW, int sh, int sw, int dh, int dw, int pad_t,
                             int pad_l, int64_t Ho, int64_t Wo, int act, float max_limit, float coef) {
  const int64_t K = C * KH * KW, hw = Ho * Wo;
  const int64_t Kp = (K + 3) / 4 * 4;
  const bool merged = (hw % 4 != 0) || hw < 128;
  const int64_t hwp = (hw + 3) / 4 * 4;
  const int64_t per_image = K * (merged ? hw : hwp) * 4;
  int64_t chunk = std::max<int64_t>(1, std::min<int64_t>(N, ctx->col_budget_bytes / std::max<int64_t>(per_image, 1)));
  chunk = std::min<int64_t>(chunk, 65535);
  const bool repack = (K % 4 != 0) || (reinterpret_cast<uintptr_t>(filter) & 15u);
  const int64_t merged_rs = (chunk * hw + 3) / 4 * 4;
  size_t off = 0;
  const size_t off_f = off; off += repack ? align_up(sizeof(float) * O * Kp, 256) : 0;
  const size_t off_col = off; off += align_up(sizeof(float) * K * (merged ? merged_rs : chunk * hwp), 256);
  const size_t off_c2 = off; off += merged ? align_up(sizeof(float) * O * merged_rs, 256) : 0;
  uint8_t *scratch = nullptr;
  MB_RETURN_IF_ERROR(mb_scratch(ctx, off, reinterpret_cast<void **>(&scratch)));
  const float *wmat = filter;
  int64_t w_rs = K;
  if (repack) {
    float *wf = reinterpret_cast<float *>(scratch + off_f);
    repack_rows_f32_kernel<<<static_cast<unsigned>(ceil_div64(O * Kp, 256)), 256, 0, ctx->stream>>>(
        filter, wf, O, static_cast<int>(K), static_cast<int>(Kp));
    MB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
    wmat = wf;
    w_rs = Kp;
  }
  float *col = reinterpret_cast<float *>(scratch + off_col);
  float *c2 = reinterpret_cast<float *>(scratch + off_c2);
  ColF32Params p;
  p.col = col;
  p.C = static_cast<int>(C); p.H = static_cast<int>(H); p.W = static_cast<int>(W);
  p.KH = static_cast<int>(KH); p.KW = static_cast<int>(KW);
  p.sh = sh; p.sw = sw; p.dh = dh; p.dw = dw; p.pad_t = pad_t; p.pad_l = pad_l;
  p.Ho = static_cast<int>(Ho); p.Wo = static_cast<int>(Wo); p.hw = static_cast<int>(hw);
  for (int64_t n0 = 0; n0 < N; n0 += chunk) {
    const int64_t nc = std::min(chunk, N - n0);
    p.in = in + n0 * C * H * W;
    p.col_rs = merged ? merged_rs : hwp;
    p.col_ns = merged ? hw : K * hwp;
    int bw = 8;  // threads along a row: the power of two that covers Wo, at most 128
    while (bw < Wo && bw < 128) bw *= 2;
    dim3 block(bw, 128 / bw);
    // a block of few useful threads (narrow or single-tap rows) takes several (channel,
    // filter row) pairs, so that its launch cost is spread over more than a handful of values
    const int rows_per_block = (C * KH >= 64 && Wo * KW < 512) ? 8 : 1;
    dim3 grid(static_cast<unsigned>(ceil_div64(Ho, block.y)),
              static_cast<unsigned>(ceil_div64(C * KH, rows_per_block)), static_cast<unsigned>(nc));
    im2col_f32_kernel<<<grid, block, 0, ctx->stream>>>(p, rows_per_block);
    MB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
    float *dst = out + n0 * O * hw;
    if (!merged) {
      // out_n [O x hw] = filter [O x K] * col_n [K x hw]
      MB_RETURN_IF_ERROR(mb_gemm_f32_strided(ctx, wmat, col, dst, bias, nc, O, hw, K, w_rs, 1, 0, hwp, 1,
                                             K * hwp, hw, 1, O * hw, act, max_limit, coef));
    } else {
      MB_RETURN_IF_ERROR(mb_gemm_f32_strided(ctx, wmat, col, c2, bias, 1, O, nc * hw, K, w_rs, 1, 0,
                                             merged_rs, 1, 0, merged_rs, 1, 0, act, max_limit, coef));
      const int64_t total = nc * O * hw;
      unmerge_f32_kernel<<<static_cast<unsigned>(ceil_div64(total, 256)), 256, 0, ctx->stream>>>(
          c2, dst, total, static_cast<int>(O), static_cast<int>(hw), merged_rs);
      MB_CUDA(ctx, cudaGetLastError());
      ctx->launches++;
    }
  }
  return MB_SUCCESS;
}

extern "C" {

int mb_gemm_f32(mb_context *ctx, const float *A, const float *B, float *C, int64_t batch,
                int64_t M, int64_t N, int64_t K, int a_col_major, int b_col_major,
                int c_col_major, int a_batched, int b_batched) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (batch < 0 || M < 0 || N < 0 || K < 0)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_gemm_f32: negative dimension");
  if (batch == 0 || M == 0 || N == 0) return MB_SUCCESS;
  if (A == nullptr || B == nullptr || C == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_gemm_f32: null operand");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  return mb_gemm_f32_strided(ctx, A, B, C, nullptr, batch, M, N, K, a_col_major ? 1 : K,
                             a_col_major ? M : 1, a_batched ? M * K : 0, b_col_major ? 1 : N,
                             b_col_major ? K : 1, b_batched ? K * N : 0, c_col_major ? 1 : N,
                             c_col_major ? M : 1, M * N, 0, 0.f, 0.f);
}

int mb_gemv_f32(mb_context *ctx, const float *lhs, const float *rhs, const float *bias,
                float *out, int64_t batch, int64_t rows, int64_t K, int lhs_batched,
                int rhs_batched) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (batch < 0 || rows < 0 || K < 0)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_gemv_f32: negative dimension");
  if (batch == 0 || rows == 0) return MB_SUCCESS;
  if (lhs == nullptr || rhs == nullptr || out == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_gemv_f32: null operand");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  // Many vectors against one matrix (FullyConnected on a batch) on the tensor cores: the
  // vectors are transposed to [K x batch] (the kernel's activation operand has the long
  // dimension contiguous), the product comes out as [rows x batch] and is transposed back.
  if (!lhs_batched && rhs_batched && batch >= 32 && batch % 4 == 0 && K % 4 == 0 && rows >= 16 &&
      batch < (1 << 30) && K < (1 << 30) && rows < (1 << 30)) {
    float *scratch = nullptr;
    const size_t xt_bytes = align_up(sizeof(float) * K * batch, 256);
    MB_RETURN_IF_ERROR(mb_scratch(ctx, xt_bytes + sizeof(float) * rows * batch, reinterpret_cast<void **>(&scratch)));
    float *xt = scratch, *ct = scratch + xt_bytes / sizeof(float);
    if (mb_gemm_f32_tc_supported(ctx, xt, lhs, batch, rows, K, batch, 0, K, 0)) {
      dim3 g1(static_cast<unsigned>(ceil_div64(K, 32)), static_cast<unsigned>(ceil_div64(batch, 32)));
      transpose_f32_kernel<<<g1, 256, 0, ctx->stream>>>(rhs, xt, static_cast<int>(batch), static_cast<int>(K));
      MB_CUDA(ctx, cudaGetLastError());
      MB_RETURN_IF_ERROR(mb_gemm_f32_tc_launch(ctx, xt, lhs, bias, ct, 1, batch, rows, K, batch, 0, K, 0, batch, 0,
                                               0, 0.f, 0.f, nullptr));
      dim3 g2(static_cast<unsigned>(ceil_div64(batch, 32)), static_cast<unsigned>(ceil_div64(rows, 32)));
      transpose_f32_kernel<<<g2, 256, 0, ctx->stream>>>(ct, out, static_cast<int>(rows), static_cast<int>(batch));
      MB_CUDA(ctx, cudaGetLastError());
      ctx->launches += 2;
      return MB_SUCCESS;
    }
  }
  int64_t chunks = std::min<int64_t>(batch, 65535);
  if (!lhs_batched)
    chunks = std::min<int64_t>(chunks, std::max<int64_t>(1, (4ll * ctx->num_sms) / ceil_div64(rows, 8)));
  const int batch_chunk = static_cast<int>(ceil_div64(batch, chunks));
  dim3 grid(static_cast<unsigned>(ceil_div64(rows, 8)),
            static_cast<unsigned>(ceil_div64(batch, batch_chunk)));
  gemv_f32_kernel<<<grid, 256, 0, ctx->stream>>>(lhs, rhs, bias, out, batch, rows, K, lhs_batched,
                                                 rhs_batched, batch_chunk);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

static int check_conv_f32(mb_context *ctx, const char *who, const float *in, const float *filter,
                          float *out, int64_t N, int64_t C, int64_t H, int64_t W, int64_t O,
                          int64_t KH, int64_t KW, int sh, int sw, int dh, int dw, int pt, int pl,
                          int64_t Ho, int64_t Wo, int act, bool *empty) {
  *empty = false;
  if (N < 0 || C < 1 || H < 1 || W < 1 || O < 1 || KH < 1 || KW < 1 || sh < 1 || sw < 1 ||
      dh < 1 || dw < 1 || pt < 0 || pl < 0 || Ho < 0 || Wo < 0)
    return mb_fail(ctx, MB_INVALID_ARGS, "%s: bad shape argument", who);
  if (!(act == 0 || act == 1 || act == 2 || act == 6))
    return mb_fail(ctx, MB_UNSUPPORTED, "%s: activation %d is not fused here", who, act);
  if (N == 0 || Ho == 0 || Wo == 0) {
    *empty = true;
    return MB_SUCCESS;
  }
  if (in == nullptr || filter == nullptr || out == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "%s: null operand", who);
  if (N * O * Ho * Wo >= (1ll << 38) || N * C * H * W >= (1ll << 38))
    return mb_fail(ctx, MB_UNSUPPORTED, "%s: tensor too large", who);
  return MB_SUCCESS;
}

int mb_conv2d_f32_nchw(mb_context *ctx, const float *in, const float *filter, const float *bias,
                       float *out, int64_t N, int64_t C, int64_t H, int64_t W, int64_t O,
                       int64_t KH, int64_t KW, int stride_h, int stride_w, int dil_h, int dil_w,
                       int pad_top, int pad_left, int64_t Ho, int64_t Wo, int activation,
                       float max_limit, float coefficient) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  bool empty;
  MB_RETURN_IF_ERROR(check_conv_f32(ctx, "mb_conv2d_f32_nchw", in, filter, out, N, C, H, W, O, KH,
                                    KW, stride_h, stride_w, dil_h, dil_w, pad_top, pad_left, Ho,
                                    Wo, activation, &empty));
  if (empty) return MB_SUCCESS;
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  if (KH == 1 && KW == 1 && stride_h == 1 && stride_w == 1 && pad_top == 0 && pad_left == 0 &&
      Ho == H && Wo == W && ((H * W) % 4 == 0 && H * W >= 128 || !ctx->use_tensor_cores)) {
    // out_n[O x HW] = filter[O x C] * in_n[C x HW] for every image n
    // (arm::Conv2dK1x1, mace/ops/arm/base/conv_2d_1x1.cc:61-68)
    const int64_t hw = H * W;
    return mb_gemm_f32_strided(ctx, filter, in, out, bias, N, O, hw, C, C, 1, 0, hw, 1, C * hw, hw,
                               1, O * hw, activation, max_limit, coefficient);
  }
  // enough work to fill tensor-core tiles: gather columns and multiply; tiny problems stay on
  // the one-thread-per-output kernel
  if (N * O * Ho * Wo * C * KH * KW >= (1ll << 18) && Ho * Wo * N >= 32 && C * KH <= 65535 &&
      Ho * Wo < (1ll << 30)) {
    return conv2d_f32_im2col(ctx, in, filter, bias, out, N, C, H, W, O, KH, KW, stride_h, stride_w, dil_h,
                             dil_w, pad_top, pad_left, Ho, Wo, activation, max_limit, coefficient);
  }
  ConvF32Params p;
  p.in = in; p.filter = filter; p.bias = bias; p.out = out;
  p.N = static_cast<int>(N); p.C = static_cast<int>(C); p.H = static_cast<int>(H); p.W = static_cast<int>(W);
  p.O = static_cast<int>(O); p.KH = static_cast<int>(KH); p.KW = static_cast<int>(KW);
  p.sh = stride_h; p.sw = stride_w; p.dh = dil_h; p.dw = dil_w; p.pad_t = pad_top; p.pad_l = pad_left;
  p.Ho = static_cast<int>(Ho); p.Wo = static_cast<int>(Wo); p.mult_ch = 1;
  p.act = activation; p.max_limit = max_limit; p.coef = coefficient;
  const int64_t total = N * O * Ho * Wo;
  conv2d_f32_direct_kernel<<<static_cast<unsigned>(ceil_div64(total, 256)), 256, 0, ctx->stream>>>(p);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

int mb_conv2d_f32_nchw_residual(mb_context *ctx, const float *in, const float *filter, const float *bias,
                                const float *residual, float *out, int64_t N, int64_t C, int64_t H,
                                int64_t W, int64_t O, int64_t KH, int64_t KW, int stride_h, int stride_w,
                                int dil_h, int dil_w, int pad_top, int pad_left, int64_t Ho, int64_t Wo,
                                int activation, float max_limit, float coefficient) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (residual == nullptr)
    return mb_conv2d_f32_nchw(ctx, in, filter, bias, out, N, C, H, W, O, KH, KW, stride_h, stride_w, dil_h,
                              dil_w, pad_top, pad_left, Ho, Wo, activation, max_limit, coefficient);
  bool empty;
  MB_RETURN_IF_ERROR(check_conv_f32(ctx, "mb_conv2d_f32_nchw_residual", in, filter, out, N, C, H, W, O, KH,
                                    KW, stride_h, stride_w, dil_h, dil_w, pad_top, pad_left, Ho, Wo,
                                    activation, &empty));
  if (empty) return MB_SUCCESS;
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  const int64_t hw = H * W;
  // 1x1 stride 1 on the tensor cores: the sum and the activation ride in the GEMM's epilogue
  if (KH == 1 && KW == 1 && stride_h == 1 && stride_w == 1 && pad_top == 0 && pad_left == 0 && Ho == H &&
      Wo == W && hw % 4 == 0 && hw >= 128 &&
      mb_gemm_f32_tc_supported(ctx, in, filter, hw, O, C, hw, C * hw, C, 0) &&
      (reinterpret_cast<uintptr_t>(residual) & 3u) == 0) {
    return mb_gemm_f32_tc_launch(ctx, in, filter, bias, out, N, hw, O, C, hw, C * hw, C, 0, hw, O * hw,
                                 activation, max_limit, coefficient, residual);
  }
  // every other shape: the convolution without activation, then sum + activation in place
  MB_RETURN_IF_ERROR(mb_conv2d_f32_nchw(ctx, in, filter, bias, out, N, C, H, W, O, KH, KW, stride_h, stride_w,
                                        dil_h, dil_w, pad_top, pad_left, Ho, Wo, 0, 0.f, 0.f));
  return mb_eltwise_act_f32(ctx, out, residual, out, N * O * Ho * Wo, 0, 0.f, 0, 0.f, 0.f, 0, activation,
                            max_limit, coefficient);
}

int mb_dwconv_f32_nchw(mb_context *ctx, const float *in, const float *filter, const float *bias,
                       float *out, int64_t N, int64_t C, int64_t H, int64_t W, int64_t mult_ch,
                       int64_t KH, int64_t KW, int stride_h, int stride_w, int dil_h, int dil_w,
                       int pad_top, int pad_left, int64_t Ho, int64_t Wo, int activation,
                       float max_limit, float coefficient) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  bool empty;
  MB_RETURN_IF_ERROR(check_conv_f32(ctx, "mb_dwconv_f32_nchw", in, filter, out, N, C, H, W,
                                    mult_ch, KH, KW, stride_h, stride_w, dil_h, dil_w, pad_top,
                                    pad_left, Ho, Wo, activation, &empty));
  if (empty) return MB_SUCCESS;
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  ConvF32Params p;
  p.in = in; p.filter = filter; p.bias = bias; p.out = out;
  p.N = static_cast<int>(N); p.C = static_cast<int>(C); p.H = static_cast<int>(H); p.W = static_cast<int>(W);
  p.O = static_cast<int>(C * mult_ch); p.KH = static_cast<int>(KH); p.KW = static_cast<int>(KW);
  p.sh = stride_h; p.sw = stride_w; p.dh = dil_h; p.dw = dil_w; p.pad_t = pad_top; p.pad_l = pad_left;
  p.Ho = static_cast<int>(Ho); p.Wo = static_cast<int>(Wo); p.mult_ch = static_cast<int>(mult_ch);
  p.act = activation; p.max_limit = max_limit; p.coef = coefficient;
  const int64_t total = N * C * mult_ch * Ho * Wo;
  dwconv_f32_kernel<<<static_cast<unsigned>(ceil_div64(total, 256)), 256, 0, ctx->stream>>>(p);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

}  // extern "C"
