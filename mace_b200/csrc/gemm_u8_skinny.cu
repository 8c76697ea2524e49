// uint8 GEMM with very few rows (M <= 16) against a row-major B [K x N]: the M = 1 and
// M = 16 cases of a MatMul whose right-hand side is a large weight matrix.
//
// Reference behaviour: MatMulFixpointImpl (mace/ops/matmul.cc:228-394) -- on x86 such a
// product stays in gemmlowp with the fixed-point output pipeline
// (mace/ops/common/gemmlowp_util.h:37-74); results here are bit-identical to mb_gemm_u8's
// other kernels.
//
// The work is streaming B once from HBM, so it is spread over all SMs by splitting BOTH N and
// K: a thread owns 4 adjacent columns and 32 consecutive k-rows.  It loads one 32-bit word per
// row (a warp reads 128 contiguous bytes), transposes 4 rows x 4 columns with byte permutes so
// that each word holds 4 consecutive k of one column, and feeds dp4a with the matching 4 bytes
// of every A row (broadcast reads from shared memory).  Column sums of B for the zero-point
// correction come from the same words.  The 8 k-slices of a block are added up in shared
// memory and written as one partial tile per block; the block that arrives last for its 128
// columns (a counter per column block, no waiting) adds the partial tiles, the corrections
// and the bias, requantizes and stores, and resets the counter for the next call.
#include <algorithm>

#include "common.cuh"

namespace {

constexpr int SK_ROWS = 32;    // k-rows per thread
constexpr int SK_COLS = 128;   // columns per block (32 lanes x 4)
constexpr int SK_WARPS = 8;    // k-slices per block

struct SkinnyParams {
  const uint8_t *A, *B;
  const int32_t *bias;
  void *C;
  int M, N, K;
  int out_is_int32, bias_per_row;
  int32_t zp_a, zp_b;
  mb_requant_params rq;
  int32_t *partial;    // [k-blocks][(MT + 1)][N]: per-block sums, last row = B's column sums
  unsigned *counters;  // [N / 128]: arrivals per column block; zero on entry and on exit
};

__device__ __forceinline__ void transpose4(const uint32_t (&w)[4], uint32_t (&t)[4]) {
  const uint32_t lo01 = __byte_perm(w[0], w[1], 0x5140), hi01 = __byte_perm(w[0], w[1], 0x7362);
  const uint32_t lo23 = __byte_perm(w[2], w[3], 0x5140), hi23 = __byte_perm(w[2], w[3], 0x7362);
  t[0] = __byte_perm(lo01, lo23, 0x5410);
  t[1] = __byte_perm(lo01, lo23, 0x7632);
  t[2] = __byte_perm(hi01, hi23, 0x5410);
  t[3] = __byte_perm(hi01, hi23, 0x7632);
}

template <int MT>
__global__ void __launch_bounds__(SK_WARPS * 32) gemm_u8_skinny_kernel(const SkinnyParams p) {
  __shared__ uint32_t a_sm[MT][SK_WARPS * SK_ROWS / 4];   // A[m][k-range of the block], 4 k per word
  extern __shared__ int4 slab[];  // [SK_WARPS][MT + 1][32 lanes]: each warp's sums, 4 columns per lane
  __shared__ int32_t rowsum[16];
  __shared__ int last_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * SK_COLS + lane * 4;
  const int kb0 = blockIdx.y * (SK_WARPS * SK_ROWS);
  const int k0 = kb0 + warp * SK_ROWS;
  const bool col_ok = n0 < p.N;
  const uint8_t *bp = p.B + static_cast<int64_t>(k0) * p.N + n0;
  // all 32 rows of the thread are requested before anything else
  uint32_t w[SK_ROWS / 4][4];
#pragma unroll
  for (int g = 0; g < SK_ROWS / 4; ++g)
#pragma unroll
    for (int r = 0; r < 4; ++r)
      w[g][r] = (col_ok && k0 + g * 4 + r < p.K)
                    ? __ldg(reinterpret_cast<const uint32_t *>(bp + static_cast<int64_t>(g * 4 + r) * p.N))
                    : 0u;
  // A slice -> shared memory (zero beyond M or K)
  for (int i = threadIdx.x; i < MT * (SK_WARPS * SK_ROWS / 4); i += blockDim.x) {
    const int m = i / (SK_WARPS * SK_ROWS / 4), kq = i % (SK_WARPS * SK_ROWS / 4);
    const int k = kb0 + kq * 4;
    uint32_t v = 0;
    if (m < p.M && k < p.K) v = __ldg(reinterpret_cast<const uint32_t *>(p.A + static_cast<int64_t>(m) * p.K + k));
    a_sm[m][kq] = v;
  }
  __syncthreads();

  int32_t acc[MT][4];
  uint32_t csum[4] = {0, 0, 0, 0};
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[m][c] = 0;
#pragma unroll
  for (int g = 0; g < SK_ROWS / 4; ++g) {
    uint32_t t[4];
    transpose4(w[g], t);
#pragma unroll
    for (int c = 0; c < 4; ++c) csum[c] = __dp4a(t[c], 0x01010101u, csum[c]);
    const int kq = warp * (SK_ROWS / 4) + g;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const uint32_t a = a_sm[m][kq];
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[m][c] = static_cast<int32_t>(__dp4a(a, t[c], static_cast<uint32_t>(acc[m][c])));
    }
  }
  // 8 k-slices -> one partial tile per block
#pragma unroll
  for (int m = 0; m < MT; ++m)
    slab[(warp * (MT + 1) + m) * 32 + lane] = make_int4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
  slab[(warp * (MT + 1) + MT) * 32 + lane] = make_int4(csum[0], csum[1], csum[2], csum[3]);
  __syncthreads();
  int4 *pt = reinterpret_cast<int4 *>(p.partial + static_cast<int64_t>(blockIdx.y) * (MT + 1) * p.N);
  for (int i = threadIdx.x; i < (MT + 1) * 32; i += blockDim.x) {
    const int r = i >> 5, l = i & 31;
    int4 t = slab[r * 32 + l];
#pragma unroll
    for (int ws = 1; ws < SK_WARPS; ++ws) {
      const int4 u = slab[(ws * (MT + 1) + r) * 32 + l];
      t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
    }
    const int n = blockIdx.x * SK_COLS + l * 4;
    if (n < p.N) pt[(static_cast<int64_t>(r) * p.N + n) >> 2] = t;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();  // cumulative: publishes the whole block's partial tile before the count
    last_flag = atomicAdd(p.counters + blockIdx.x, 1u) == gridDim.y - 1 ? 1 : 0;
    __threadfence();
  }
  __syncthreads();
  if (!last_flag) return;
  // ---- the last block for these 128 columns finishes them ----
  // row sums of A (for B's zero point): warp w sums rows w, w + 8, ...
  for (int m = warp; m < p.M; m += SK_WARPS) {
    uint32_t s = 0;
    for (int k = lane * 4; k < p.K; k += 128)
      s = __dp4a(__ldg(reinterpret_cast<const uint32_t *>(p.A + static_cast<int64_t>(m) * p.K + k)), 0x01010101u, s);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) rowsum[m] = static_cast<int32_t>(s);
  }
  __syncthreads();
  const int32_t kzz = static_cast<int32_t>(static_cast<uint32_t>(p.K) * static_cast<uint32_t>(p.zp_a) *
                                           static_cast<uint32_t>(p.zp_b));
  const int kblocks = gridDim.y;
  const int64_t tile_stride = static_cast<int64_t>(MT + 1) * p.N;
  for (int i = threadIdx.x; i < p.M * SK_COLS; i += blockDim.x) {
    const int m = i / SK_COLS, c = i % SK_COLS;
    const int n = blockIdx.x * SK_COLS + c;
    if (n >= p.N) continue;
    int32_t raw = 0, colsum = 0;
    const int32_t *pr = p.partial + static_cast<int64_t>(m) * p.N + n;
    const int32_t *pc = p.partial + static_cast<int64_t>(MT) * p.N + n;
    int kb = 0;
    for (; kb + 8 <= kblocks; kb += 8) {  // 16 independent loads in flight
      int32_t a[8], b[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        a[u] = __ldcg(pr + (kb + u) * tile_stride);
        b[u] = __ldcg(pc + (kb + u) * tile_stride);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        raw += a[u];
        colsum += b[u];
      }
    }
    for (; kb < kblocks; ++kb) {
      raw += __ldcg(pr + kb * tile_stride);
      colsum += __ldcg(pc + kb * tile_stride);
    }
    int32_t v = raw - p.zp_a * colsum - p.zp_b * rowsum[m] + kzz;
    if (p.bias != nullptr) v += p.bias[p.bias_per_row ? m : n];
    if (p.out_is_int32) static_cast<int32_t *>(p.C)[static_cast<int64_t>(m) * p.N + n] = v;
    else static_cast<uint8_t *>(p.C)[static_cast<int64_t>(m) * p.N + n] = static_cast<uint8_t>(mb_requant_fast(v, p.rq));
  }
  if (threadIdx.x == 0) p.counters[blockIdx.x] = 0;
}

}  // namespace

// Whether the skinny kernel takes this problem: one batch entry, A k-contiguous, B row-major.
bool mb_gemm_u8_skinny_supported(int64_t batch, int64_t M, int64_t N, int64_t K, bool a_mn, bool b_mn,
                                 const void *A, const void *B) {
  return batch == 1 && M >= 1 && M <= 16 && !a_mn && b_mn && N % 4 == 0 && K % 4 == 0 && N >= 512 &&
         K >= 256 && N < (1ll << 30) && K < (1ll << 30) && 255ll * 255 * K < (1ll << 31) &&
         ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 3u) == 0;
}

int mb_gemm_u8_skinny_launch(mb_context *ctx, const uint8_t *A, const uint8_t *B, const int32_t *bias,
                             void *C, int out_is_int32, int64_t M, int64_t N, int64_t K, int32_t zp_a,
                             int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c, int bias_per_row) {
  const int MT = M <= 1 ? 1 : M <= 4 ? 4 : M <= 8 ? 8 : 16;
  const int64_t col_blocks = ceil_div64(N, SK_COLS);
  const int64_t k_blocks = ceil_div64(K, SK_WARPS * SK_ROWS);
  // counters: a small buffer of their own that is zero between calls (the kernel resets them)
  const size_t need = sizeof(unsigned) * col_blocks;
  if (ctx->skinny_ws_bytes < need) {
    if (ctx->capturing)
      return mb_fail(ctx, MB_RUNTIME_ERROR, "few-row GEMM counters would grow during graph capture");
    if (ctx->skinny_ws != nullptr) {
      MB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      MB_CUDA(ctx, cudaFree(ctx->skinny_ws));
      ctx->skinny_ws = nullptr;
      ctx->skinny_ws_bytes = 0;
    }
    const size_t want = std::max<size_t>(need, 4096);
    MB_CUDA(ctx, cudaMalloc(&ctx->skinny_ws, want));
    ctx->skinny_ws_bytes = want;
    MB_CUDA(ctx, cudaMemsetAsync(ctx->skinny_ws, 0, want, ctx->stream));
  }
  int32_t *partial = nullptr;
  MB_RETURN_IF_ERROR(mb_scratch(ctx, sizeof(int32_t) * k_blocks * (MT + 1) * N,
                                reinterpret_cast<void **>(&partial)));
  SkinnyParams p;
  p.A = A; p.B = B; p.bias = bias; p.C = C;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.out_is_int32 = out_is_int32; p.bias_per_row = bias_per_row;
  p.zp_a = zp_a; p.zp_b = zp_b;
  p.rq = mb_make_requant(mult, shift, zp_c);
  p.partial = partial;
  p.counters = static_cast<unsigned *>(ctx->skinny_ws);
  const dim3 grid(static_cast<unsigned>(col_blocks),
                  static_cast<unsigned>(k_blocks));
  if (MT == 16 && !(ctx->func_attr_mask & (1ull << 45))) {  // 68 KB of shared memory
    MB_CUDA(ctx, cudaFuncSetAttribute(gemm_u8_skinny_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(SK_WARPS * 17 * 32 * sizeof(int4))));
    ctx->func_attr_mask |= (1ull << 45);
  }
  switch (MT) {
    case 1: gemm_u8_skinny_kernel<1><<<grid, SK_WARPS * 32, SK_WARPS * (1 + 1) * 32 * sizeof(int4), ctx->stream>>>(p); break;
    case 4: gemm_u8_skinny_kernel<4><<<grid, SK_WARPS * 32, SK_WARPS * (4 + 1) * 32 * sizeof(int4), ctx->stream>>>(p); break;
    case 8: gemm_u8_skinny_kernel<8><<<grid, SK_WARPS * 32, SK_WARPS * (8 + 1) * 32 * sizeof(int4), ctx->stream>>>(p); break;
    default: gemm_u8_skinny_kernel<16><<<grid, SK_WARPS * 32, SK_WARPS * (16 + 1) * 32 * sizeof(int4), ctx->stream>>>(p); break;
  }
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}
