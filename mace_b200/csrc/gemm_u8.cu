// mb_gemm_u8: argument checks, operand preparation (row/column byte sums for
// the zero-point correction, optional transposes) and the choice between the
// tensor-core kernel (gemm_u8_tc.cu) and a CUDA-core kernel that takes any
// layout, alignment and depth.
//
// Reference behaviour: MatMulFixpointImpl (mace/ops/matmul.cc:228-394) and the
// GEMM of the quantized Conv2D (mace/ops/conv_2d.cc:301-315).
#include <algorithm>

#include "common.cuh"

bool mb_gemm_u8_tc_supported(const mb_context *ctx, const void *A, const void *B, int64_t M,
                             int64_t N, int64_t K, bool a_mn, bool b_mn, int a_batched,
                             int b_batched);
int mb_gemm_u8_tc_launch(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                         const uint32_t *sum_a, const uint32_t *sum_b, const int32_t *bias,
                         void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N,
                         int64_t K, bool a_mn, bool b_mn, int a_batched, int b_batched,
                         int32_t zp_a, int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c,
                         int bias_per_row);

namespace {

// ---- CUDA-core GEMM: any major order, any size --------------------------------
// 64 x 64 output tile per 256-thread block, 4 x 4 outputs per thread.  Operands
// are read element-wise with their own strides, the zero points are subtracted
// on load, so no correction terms and no overflow for any depth whose true
// result fits int32.
constexpr int GT = 64;   // tile edge
constexpr int GK = 32;   // depth per step

struct GenericParams {
  const uint8_t *A, *B;
  const int32_t *bias;
  void *C;
  int64_t M, N, K;
  int64_t a_rs, a_cs;  // strides of A(m,k): m * a_rs + k * a_cs
  int64_t b_rs, b_cs;  // strides of B(k,n): k * b_rs + n * b_cs
  int64_t a_bs, b_bs;  // batch strides (0 when not batched)
  int32_t zp_a, zp_b;
  mb_requant_params rq;
  int out_is_int32, bias_per_row;
};

__global__ void __launch_bounds__(256) gemm_u8_generic_kernel(const GenericParams p) {
  __shared__ int16_t As[GK][GT + 2];
  __shared__ int16_t Bs[GK][GT + 2];
  const int b = blockIdx.z;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * GT;
  const int64_t n0 = static_cast<int64_t>(blockIdx.x) * GT;
  const uint8_t *A = p.A + b * p.a_bs;
  const uint8_t *B = p.B + b * p.b_bs;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  int32_t acc[4][4] = {};
  for (int64_t k0 = 0; k0 < p.K; k0 += GK) {
    for (int i = threadIdx.x; i < GK * GT; i += 256) {
      // pick the fastest-varying index so that loads coalesce for either major
      int kk, mm;
      if (p.a_cs == 1) { kk = i % GK; mm = i / GK; } else { mm = i % GT; kk = i / GT; }
      const int64_t m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < p.M && k < p.K)
                       ? static_cast<int16_t>(static_cast<int32_t>(A[m * p.a_rs + k * p.a_cs]) - p.zp_a)
                       : 0;
      int nn;
      if (p.b_cs == 1) { nn = i % GT; kk = i / GT; } else { kk = i % GK; nn = i / GK; }
      const int64_t n = n0 + nn;
      const int64_t kb = k0 + kk;
      Bs[kk][nn] = (n < p.N && kb < p.K)
                       ? static_cast<int16_t>(static_cast<int32_t>(B[kb * p.b_rs + n * p.b_cs]) - p.zp_b)
                       : 0;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < GK; ++kk) {
      int32_t a[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * bv[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      int32_t v = acc[i][j];
      if (p.bias != nullptr) v += p.bias_per_row ? p.bias[m] : p.bias[n];
      const int64_t idx = (static_cast<int64_t>(b) * p.M + m) * p.N + n;
      if (p.out_is_int32) {
        static_cast<int32_t *>(p.C)[idx] = v;
      } else {
        static_cast<uint8_t *>(p.C)[idx] =
            static_cast<uint8_t>(mb_requant_fast(v, p.rq));
      }
    }
  }
}

// ---- transpose [rows x cols] -> [cols x rows] bytes ------------------------------
__global__ void __launch_bounds__(256) transpose_u8_kernel(const uint8_t *__restrict__ in,
                                                           uint8_t *__restrict__ out,
                                                           int64_t rows, int64_t cols) {
  __shared__ uint8_t tile[64][65];
  const int64_t batch_off = static_cast<int64_t>(blockIdx.z) * rows * cols;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * 64, c0 = static_cast<int64_t>(blockIdx.x) * 64;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int r = i >> 6, c = i & 63;
    tile[r][c] = (r0 + r < rows && c0 + c < cols) ? in[batch_off + (r0 + r) * cols + c0 + c] : 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int c = i >> 6, r = i & 63;
    if (r0 + r < rows && c0 + c < cols) out[batch_off + (c0 + c) * rows + r0 + r] = tile[r][c];
  }
}

int launch_transpose(mb_context *ctx, const uint8_t *in, uint8_t *out, int64_t nb, int64_t rows,
                     int64_t cols) {
  dim3 grid(static_cast<unsigned>(ceil_div64(cols, 64)), static_cast<unsigned>(ceil_div64(rows, 64)),
            static_cast<unsigned>(nb));
  transpose_u8_kernel<<<grid, 256, 0, ctx->stream>>>(in, out, rows, cols);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

int launch_generic(mb_context *ctx, const uint8_t *A, const uint8_t *B, const int32_t *bias,
                   void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N, int64_t K,
                   bool a_mn, bool b_mn, int a_batched, int b_batched, int32_t zp_a,
                   int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c, int bias_per_row) {
  GenericParams p;
  p.A = A; p.B = B; p.bias = bias; p.C = C;
  p.M = M; p.N = N; p.K = K;
  // A K-major: (m,k) at m*K + k.  A MN-major: (m,k) at k*M + m.
  p.a_rs = a_mn ? 1 : K; p.a_cs = a_mn ? M : 1;
  // B MN-major (row-major K x N): (k,n) at k*N + n.  B K-major: n*K + k.
  p.b_rs = b_mn ? N : 1; p.b_cs = b_mn ? 1 : K;
  p.a_bs = a_batched ? M * K : 0; p.b_bs = b_batched ? K * N : 0;
  p.zp_a = zp_a; p.zp_b = zp_b;
  p.rq = mb_make_requant(mult, shift, zp_c);
  p.out_is_int32 = out_is_int32; p.bias_per_row = bias_per_row;
  const int64_t gx = ceil_div64(N, GT), gy = ceil_div64(M, GT);
  if (gy > 65535 || batch > 65535)
    return mb_fail(ctx, MB_UNSUPPORTED, "generic GEMM: M or batch too large for this path");
  dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(batch));
  gemm_u8_generic_kernel<<<grid, 256, 0, ctx->stream>>>(p);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

}  // namespace

bool mb_gemm_u8_skinny_supported(int64_t batch, int64_t M, int64_t N, int64_t K, bool a_mn, bool b_mn,
                                 const void *A, const void *B);
int mb_gemm_u8_skinny_launch(mb_context *ctx, const uint8_t *A, const uint8_t *B, const int32_t *bias,
                             void *C, int out_is_int32, int64_t M, int64_t N, int64_t K, int32_t zp_a,
                             int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c, int bias_per_row);

int mb_operand_sums_slices(const mb_context *ctx, bool mn, int64_t nb, int64_t K, int64_t cols);
int mb_gemm_u8_tc_launch_sliced(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                                const uint32_t *sum_a, const uint32_t *sum_b, int sum_a_slices, int sum_b_slices,
                                const int32_t *bias, void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N,
                                int64_t K, bool a_mn, bool b_mn, int a_batched, int b_batched,
                                int32_t zp_a, int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c,
                                int bias_per_row);
int mb_operand_sums_launch(mb_context *ctx, const uint8_t *A, bool a_mn, int64_t nb_a, int64_t M, uint32_t *sum_a,
                           const uint8_t *B, bool b_mn, int64_t nb_b, int64_t N, uint32_t *sum_b, int64_t K,
                           int k_split);
int mb_gemm_u8_tc_launch_splitk(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                                const uint32_t *sum_a, const uint32_t *sum_b, int sum_a_slices, int sum_b_slices,
                                int32_t *parts, int k_split, int bn, int64_t M, int64_t N, int64_t K, bool a_mn,
                                bool b_mn, int32_t zp_a, int32_t zp_b);

namespace {

// ---- few output tiles, long depth: the depth cut into runs ----------------------------
// A product of 128 rows against a 4096 x 4096 matrix has 32 output tiles for 148 SMs, and each
// of the 32 pulls a megabyte through one SM.  Cutting the depth into S runs gives S times the
// CTAs, each streaming 1/S of the bytes; the S exact int32 partial results (zero-point terms
// included: they are linear in the depth) are added here, then bias and the fixed-point
// output stage as in the GEMM's own epilogue (mace/ops/common/gemmlowp_util.h:37-74).
struct SplitReduceParams {
  const int32_t *parts;   // [splits][M][N]
  const int32_t *bias;
  void *C;
  int64_t M, N;
  int splits, bias_per_row, out_is_int32;
  mb_requant_params rq;
};

template <int VEC>
__global__ void __launch_bounds__(256) gemm_u8_split_reduce_kernel(const SplitReduceParams p) {
  mb_grid_dep_launch();
  mb_grid_dep_wait();
  const int64_t total = p.M * p.N / VEC;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t e = i * VEC;
    const int64_t m = e / p.N, n = e % p.N;
    int32_t acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0;
    for (int s = 0; s < p.splits; ++s) {
      const int32_t *src = p.parts + s * p.M * p.N + e;
      if (VEC == 4) {
        const int4 v = *reinterpret_cast<const int4 *>(src);
        acc[0] += v.x; acc[1 % VEC] += v.y; acc[2 % VEC] += v.z; acc[3 % VEC] += v.w;
      } else {
        acc[0] += src[0];
      }
    }
    if (p.bias != nullptr) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] += p.bias[p.bias_per_row ? m : n + j];
    }
    if (p.out_is_int32) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) static_cast<int32_t *>(p.C)[e + j] = acc[j];
    } else if (VEC == 4) {
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < VEC; ++j) w |= mb_requant_fast(acc[j], p.rq) << (8 * j);
      *reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(p.C) + e) = w;
    } else {
      static_cast<uint8_t *>(p.C)[e] = static_cast<uint8_t>(mb_requant_fast(acc[0], p.rq));
    }
  }
}

// The number of runs for this shape (1: do not cut), and the tile width to run them with.
int split_k_choice(const mb_context *ctx, int64_t batch, int64_t M, int64_t N, int64_t K, int *bn) {
  if (!ctx->split_k || batch != 1 || K < 2048) return 1;
  *bn = N >= 128 ? 128 : 64;
  const int64_t tiles = ceil_div64(M, 128) * ceil_div64(N, *bn);
  int best = 1;
  for (int s : {2, 4, 8}) {
    if (tiles * s > ctx->num_sms) break;
    if (K % (static_cast<int64_t>(s) * 128) != 0 || K / s < 512) break;
    best = s;
  }
  // two runs do not pay for the extra kernel and the int32 round trip (measured at
  // M = 256, K = N = 4096: 15.2 us against 13.9 us undivided)
  return best >= 4 ? best : 1;
}

}  // namespace

// Row-major-C GEMM on device operands; a_mn / b_mn as in mb_gemm_u8_tc_launch.
int mb_gemm_u8_rowmajor(mb_context *ctx, const uint8_t *A, const uint8_t *B, const int32_t *bias,
                        void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N,
                        int64_t K, bool a_mn, bool b_mn, int a_batched, int b_batched,
                        int32_t zp_a, int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c,
                        int bias_per_row) {
  const bool aligned16 =
      ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15u) == 0;
  bool use_tc = ctx->use_tensor_cores && ctx->encode_tiled != nullptr && aligned16 &&
                K % 16 == 0 && K <= 33000 && M >= 1 && N >= 1;
  // A few rows against a large row-major B: stream B once over all SMs with CUDA cores.  From
  // two rows on the tensor-core kernel over depth runs is faster where it applies (measured at
  // K = N = 4096: 11.4 us against 12.4 at M = 2, 11.4 against 14.0 at M = 4, 11.7 against 28.8 at
  // M = 16; a tie, 11.4 / 11.2, at M = 1).
  if (ctx->use_tensor_cores && M <= ctx->skinny_max_m && mb_gemm_u8_skinny_supported(batch, M, N, K, a_mn, b_mn, A, B)) {
    int bn_unused = 0;
    const bool runs_apply = M >= ctx->runs_min_m && use_tc && !(a_mn && !(ctx->use_mn_major && M % 16 == 0)) &&
                            !(b_mn && !(ctx->use_mn_major && N % 16 == 0)) &&
                            split_k_choice(ctx, batch, M, N, K, &bn_unused) > 1;
    if (!runs_apply)
      return mb_gemm_u8_skinny_launch(ctx, A, B, bias, C, out_is_int32, M, N, K, zp_a, zp_b, mult, shift,
                                      zp_c, bias_per_row);
  }
  // How each operand reaches the tensor core: natively in its own major, or
  // through a K-major copy in scratch.
  bool a_copy = false, b_copy = false;
  if (use_tc) {
    if (a_mn && !(ctx->use_mn_major && M % 16 == 0)) a_copy = true;
    if (b_mn && !(ctx->use_mn_major && N % 16 == 0)) b_copy = true;
  }
  if (!use_tc) {
    return launch_generic(ctx, A, B, bias, C, out_is_int32, batch, M, N, K, a_mn, b_mn,
                          a_batched, b_batched, zp_a, zp_b, mult, shift, zp_c, bias_per_row);
  }
  const int64_t nb_a = a_batched ? batch : 1, nb_b = b_batched ? batch : 1;
  int split_bn = 0;
  const int splits = (a_copy || b_copy) ? 1 : split_k_choice(ctx, batch, M, N, K, &split_bn);
  if (splits > 1 && mb_gemm_u8_tc_supported(ctx, A, B, M, N, K / splits, a_mn, b_mn, 0, 0)) {
    const int64_t Ks = K / splits;
    // runs no longer than 1024 with a K-major A: the kernel sums the bytes of its own tiles
    const bool fused = !a_mn && Ks <= 1024;
    const bool want_a = zp_b != 0 && !fused, want_b = zp_a != 0 && !fused;
    const int sl_a = want_a ? mb_operand_sums_slices(ctx, a_mn, splits, Ks, M) : 1;
    const int sl_b = want_b ? mb_operand_sums_slices(ctx, b_mn, splits, Ks, N) : 1;
    size_t off = 0;
    const size_t off_parts = off; off += align_up(sizeof(int32_t) * splits * M * N, 256);
    const size_t off_sa = off; off += want_a ? align_up(sizeof(uint32_t) * splits * M * sl_a, 256) : 0;
    const size_t off_sb = off; off += want_b ? align_up(sizeof(uint32_t) * splits * N * sl_b, 256) : 0;
    uint8_t *scratch = nullptr;
    MB_RETURN_IF_ERROR(mb_scratch(ctx, off, reinterpret_cast<void **>(&scratch)));
    int32_t *parts = reinterpret_cast<int32_t *>(scratch + off_parts);
    uint32_t *sum_a = want_a ? reinterpret_cast<uint32_t *>(scratch + off_sa) : nullptr;
    uint32_t *sum_b = want_b ? reinterpret_cast<uint32_t *>(scratch + off_sb) : nullptr;
    if (want_a || want_b)
      MB_RETURN_IF_ERROR(mb_operand_sums_launch(ctx, A, a_mn, 1, M, sum_a, B, b_mn, 1, N, sum_b, K, splits));
    ctx->pdl_next_gemm = (want_a || want_b) ? 1 : 0;
    MB_RETURN_IF_ERROR(mb_gemm_u8_tc_launch_splitk(ctx, A, B, sum_a, sum_b, sl_a, sl_b, parts, splits, split_bn, M, N,
                                                   K, a_mn, b_mn, zp_a, zp_b));
    SplitReduceParams rp;
    rp.parts = parts; rp.bias = bias; rp.C = C; rp.M = M; rp.N = N;
    rp.splits = splits; rp.bias_per_row = bias_per_row; rp.out_is_int32 = out_is_int32;
    rp.rq = mb_make_requant(mult, shift, zp_c);
    const bool vec4 = N % 4 == 0 && (reinterpret_cast<uintptr_t>(C) & 3u) == 0;
    const int64_t work = M * N / (vec4 ? 4 : 1);
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(ceil_div64(work, 256), 8ll * ctx->num_sms));
    if (vec4) {
      MB_CUDA(ctx, mb_launch_chained(ctx, gemm_u8_split_reduce_kernel<4>, dim3(grid), dim3(256), 0, rp));
    } else {
      MB_CUDA(ctx, mb_launch_chained(ctx, gemm_u8_split_reduce_kernel<1>, dim3(grid), dim3(256), 0, rp));
    }
    MB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
    return MB_SUCCESS;
  }
  // A K-major A with K <= 1024 (B in either order): the tensor-core kernel sums the operand
  // bytes itself from the tiles it has in shared memory.
  // (option pair = 2, the CTA-pair kernel wherever it can run, takes its sums from the sums kernel)
  const bool fused_sums = !(a_mn && !a_copy) && K <= 1024 && ctx->pair_gemm != 2;
  const bool need_sum_a = zp_b != 0 && !fused_sums, need_sum_b = zp_a != 0 && !fused_sums;
  size_t off = 0;
  // (an operand that reaches the tensor core MN-major gets its column sums as a few partial rows)
  const int sl_a = need_sum_a ? mb_operand_sums_slices(ctx, a_mn && !a_copy, nb_a, K, M) : 1;
  const int sl_b = need_sum_b ? mb_operand_sums_slices(ctx, b_mn && !b_copy, nb_b, K, N) : 1;
  const size_t off_sum_a = off; off += need_sum_a ? align_up(sizeof(uint32_t) * nb_a * M * sl_a, 256) : 0;
  const size_t off_sum_b = off; off += need_sum_b ? align_up(sizeof(uint32_t) * nb_b * N * sl_b, 256) : 0;
  const size_t off_at = off; off += a_copy ? align_up(nb_a * M * K, 256) : 0;
  const size_t off_bt = off; off += b_copy ? align_up(nb_b * N * K, 256) : 0;

  uint8_t *scratch = nullptr;
  if (off > 0) MB_RETURN_IF_ERROR(mb_scratch(ctx, off, reinterpret_cast<void **>(&scratch)));
  uint32_t *sum_a = need_sum_a ? reinterpret_cast<uint32_t *>(scratch + off_sum_a) : nullptr;
  uint32_t *sum_b = need_sum_b ? reinterpret_cast<uint32_t *>(scratch + off_sum_b) : nullptr;
  const uint8_t *a_use = A, *b_use = B;
  bool a_mn_use = a_mn, b_mn_use = b_mn;
  if (a_copy) {
    // MN-major A is [K x M]; its transpose [M x K] is K-major.
    MB_RETURN_IF_ERROR(launch_transpose(ctx, A, scratch + off_at, nb_a, K, M));
    a_use = scratch + off_at;
    a_mn_use = false;
  }
  if (b_copy) {
    MB_RETURN_IF_ERROR(launch_transpose(ctx, B, scratch + off_bt, nb_b, K, N));
    b_use = scratch + off_bt;
    b_mn_use = false;
  }
  // both operands' sums in one launch (see operand_sums.cu)
  if (need_sum_a || need_sum_b)
    MB_RETURN_IF_ERROR(mb_operand_sums_launch(ctx, a_use, a_mn_use, nb_a, M, sum_a, b_use, b_mn_use, nb_b, N, sum_b, K, 1));
  if (!mb_gemm_u8_tc_supported(ctx, a_use, b_use, M, N, K, a_mn_use, b_mn_use, a_batched,
                               b_batched)) {
    return launch_generic(ctx, A, B, bias, C, out_is_int32, batch, M, N, K, a_mn, b_mn,
                          a_batched, b_batched, zp_a, zp_b, mult, shift, zp_c, bias_per_row);
  }
  // The operand-sum kernel was the last launch: the GEMM may overlap it (programmatic
  // dependent launch); its operands were complete before that kernel started.
  ctx->pdl_next_gemm = (need_sum_a || need_sum_b) ? 1 : 0;
  return mb_gemm_u8_tc_launch_sliced(ctx, a_use, b_use, sum_a, sum_b, sl_a, sl_b, bias, C, out_is_int32, batch, M,
                                     N, K, a_mn_use, b_mn_use, a_batched, b_batched, zp_a, zp_b, mult,
                                     shift, zp_c, bias_per_row);
}

extern "C" int mb_gemm_u8(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                          const int32_t *bias, void *C, int out_is_int32, int64_t batch,
                          int64_t M, int64_t N, int64_t K, int a_col_major, int b_col_major,
                          int c_col_major, int a_batched, int b_batched, int32_t zp_a,
                          int32_t zp_b, int32_t multiplier, int32_t right_shift, int32_t zp_c,
                          int bias_per_row) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (batch < 0 || M < 0 || N < 0 || K < 0)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_gemm_u8: negative dimension");
  if (batch == 0 || M == 0 || N == 0) return MB_SUCCESS;  // empty output
  if (A == nullptr || B == nullptr || C == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_gemm_u8: null operand");
  if (!out_is_int32) {
    // GetOutputMultiplierAndShift (mace/core/quantize.h:116-126) yields a
    // multiplier in [2^30, 2^31) and a right shift >= 0; RoundingDivideByPOT
    // is defined for shifts up to 31.
    if (multiplier <= 0 || right_shift < 0 || right_shift > 31)
      return mb_fail(ctx, MB_INVALID_ARGS, "mb_gemm_u8: bad multiplier %d / shift %d",
                     multiplier, right_shift);
    if (zp_c < 0 || zp_c > 255)
      return mb_fail(ctx, MB_INVALID_ARGS, "mb_gemm_u8: output zero point %d outside uint8", zp_c);
  }
  if (K == 0) {
    // Empty depth: the accumulator is zero, the pipeline still applies.
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_gemm_u8: K == 0");
  }
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  // A(m,k) is K-major unless a_col_major; B(k,n) is K-major iff b_col_major.
  if (!c_col_major) {
    return mb_gemm_u8_rowmajor(ctx, A, B, bias, C, out_is_int32, batch, M, N, K,
                               a_col_major != 0, b_col_major == 0, a_batched, b_batched, zp_a,
                               zp_b, multiplier, right_shift, zp_c, bias_per_row);
  }
  // Column-major C (M x N) is row-major C^T (N x M) = B^T * A^T: swap the
  // roles of the operands.  A'(n,k) = B(k,n) is MN-major iff B is; likewise B'.
  return mb_gemm_u8_rowmajor(ctx, B, A, bias, C, out_is_int32, batch, N, M, K,
                             /*a_mn=*/b_col_major == 0, /*b_mn=*/a_col_major != 0, b_batched,
                             a_batched, zp_b, zp_a, multiplier, right_shift, zp_c,
                             bias != nullptr ? !bias_per_row : 0);
}
