// fp32 3x3 stride-1 convolution by Winograd's minimal filtering, NCHW.
//
// Reference behaviour: arm::Conv2dK3x3Winograd<float>
// (mace/ops/arm/base/conv_2d_3x3_winograd.cc:31-787): output tiles of 6x6
// (8x8 input tiles, F(6,3)) when the input is larger than 16x16, else 2x2
// (4x4 input tiles, F(2,3)); filter transform U = G g G^T once per weight,
// input transform V = B^T d B, T = 64 (or 16) independent products
// M_t = U_t [O x C] * V_t [C x tiles], output transform Y = A^T M A, then
// bias and activation (separate passes in the CPU operator, fused here).
// The transform matrices are the ones in that file's comments (:311-328,
// :487-504, :684-697).
//
// Differences in organisation, not in arithmetic:
//  * no padded copies of input or output: the transforms read zeros outside the
//    image and write only inside it;
//  * V and M are laid out [T][C][N*tiles] and [T][O][N*tiles], so that each of
//    the T products is ONE GEMM over all images (the CPU code runs T GEMMs per
//    image);
//  * the product runs as a strided-batched GEMM.
#include "common.cuh"

int mb_gemm_f32_strided(mb_context *ctx, const float *A, const float *B, float *C,
                        const float *bias_per_row, int64_t batch, int64_t M, int64_t N, int64_t K,
                        int64_t a_rs, int64_t a_cs, int64_t a_bs, int64_t b_rs, int64_t b_cs,
                        int64_t b_bs, int64_t c_rs, int64_t c_cs, int64_t c_bs, int act,
                        float max_limit, float coef);

namespace {

struct WinoParams {
  const float *in;
  const float *bias;
  float *out;
  float *V;        // [T][C][N*tiles]
  const float *Mx; // [T][O][N*tiles]
  int N, C, H, W, O, pad_t, pad_l, Ho, Wo, th, tw;
  int act;
  float max_limit, coef;
  // bytes from one transform position to the next in V and in M (below 2^32: the host checks)
  uint32_t v_pos_bytes, m_pos_bytes;
};

// Element `pos` positions further on: one 32 x 32 -> 64-bit multiply-add per address.
__device__ __forceinline__ float *at_pos(float *base, int pos, uint32_t pos_bytes) {
  return reinterpret_cast<float *>(reinterpret_cast<char *>(base) +
                                   static_cast<uint64_t>(static_cast<uint32_t>(pos)) * pos_bytes);
}
__device__ __forceinline__ const float *at_pos(const float *base, int pos, uint32_t pos_bytes) {
  return reinterpret_cast<const float *>(reinterpret_cast<const char *>(base) +
                                         static_cast<uint64_t>(static_cast<uint32_t>(pos)) * pos_bytes);
}

__device__ __forceinline__ float act_apply(float x, int act, float max_limit, float coef) {
  switch (act) {
    case 1: return fmaxf(0.f, x);
    case 2: return fmaxf(0.f, fminf(max_limit, x));
    case 6: return fmaxf(x, 0.f) + fminf(x, 0.f) * coef;
    default: return x;
  }
}

// ---- filter transforms: OIHW -> U[T][O][C] ------------------------------------------
__global__ void __launch_bounds__(256)
wino_filter_2x2_kernel(const float *__restrict__ f, float *__restrict__ U, int C, int O) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= O * C) return;
  const float *g = f + static_cast<int64_t>(idx) * 9;
  const int64_t stride = static_cast<int64_t>(O) * C;
  const float g0 = g[0], g1 = g[1], g2 = g[2], g3 = g[3], g4 = g[4], g5 = g[5], g6 = g[6], g7 = g[7],
              g8 = g[8];
  float s[16];
  s[0] = g0;
  s[1] = (g0 + g2 + g1) * 0.5f;
  s[2] = (g0 + g2 - g1) * 0.5f;
  s[3] = g2;
  s[4] = (g0 + g6 + g3) * 0.5f;
  s[5] = ((g0 + g6 + g3) + (g2 + g8 + g5) + (g1 + g7 + g4)) * 0.25f;
  s[6] = ((g0 + g6 + g3) + (g2 + g8 + g5) - (g1 + g7 + g4)) * 0.25f;
  s[7] = (g2 + g8 + g5) * 0.5f;
  s[8] = (g0 + g6 - g3) * 0.5f;
  s[9] = ((g0 + g6 - g3) + (g2 + g8 - g5) + (g1 + g7 - g4)) * 0.25f;
  s[10] = ((g0 + g6 - g3) + (g2 + g8 - g5) - (g1 + g7 - g4)) * 0.25f;
  s[11] = (g2 + g8 - g5) * 0.5f;
  s[12] = g6;
  s[13] = (g6 + g8 + g7) * 0.5f;
  s[14] = (g6 + g8 - g7) * 0.5f;
  s[15] = g8;
#pragma unroll
  for (int i = 0; i < 16; ++i) U[idx + i * stride] = s[i];
}

__global__ void __launch_bounds__(256)
wino_filter_6x6_kernel(const float *__restrict__ f, float *__restrict__ U, int C, int O) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= O * C) return;
  const float G[8][3] = {{1.0f, 0.0f, 0.0f},
                         {-2.0f / 9, -2.0f / 9, -2.0f / 9},
                         {-2.0f / 9, 2.0f / 9, -2.0f / 9},
                         {1.0f / 90, 1.0f / 45, 2.0f / 45},
                         {1.0f / 90, -1.0f / 45, 2.0f / 45},
                         {1.0f / 45, 1.0f / 90, 1.0f / 180},
                         {1.0f / 45, -1.0f / 90, 1.0f / 180},
                         {0.0f, 0.0f, 1.0f}};
  const float *g = f + static_cast<int64_t>(idx) * 9;
  const int64_t stride = static_cast<int64_t>(O) * C;
  float s[3][8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s[0][i] = g[0] * G[i][0] + g[1] * G[i][1] + g[2] * G[i][2];
    s[1][i] = g[3] * G[i][0] + g[4] * G[i][1] + g[5] * G[i][2];
    s[2][i] = g[6] * G[i][0] + g[7] * G[i][1] + g[8] * G[i][2];
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j)
      U[idx + (i * 8 + j) * stride] = G[i][0] * s[0][j] + G[i][1] * s[1][j] + G[i][2] * s[2][j];
}

// One pass of B^T (8 points) and of A^T (8 -> 6 points) for F(6,3).
__device__ __forceinline__ void bt8(const float d[8], float o[8]) {
  o[0] = d[0] - d[6] + (d[4] - d[2]) * 5.25f;
  o[7] = d[7] - d[1] + (d[3] - d[5]) * 5.25f;
  float u = d[2] + d[6] - d[4] * 4.25f;
  float v = d[1] + d[5] - d[3] * 4.25f;
  o[1] = u + v;
  o[2] = u - v;
  u = d[6] + d[2] * 0.25f - d[4] * 1.25f;
  v = d[1] * 0.5f - d[3] * 2.5f + d[5] * 2.f;
  o[3] = u + v;
  o[4] = u - v;
  u = d[6] + (d[2] - d[4] * 1.25f) * 4.f;
  v = d[1] * 2.f - d[3] * 2.5f + d[5] * 0.5f;
  o[5] = u + v;
  o[6] = u - v;
}

__device__ __forceinline__ void at8(const float d[8], float o[6]) {
  const float u = d[1] + d[2], v = d[1] - d[2], w = d[3] + d[4], x = d[3] - d[4], y = d[5] + d[6],
              z = d[5] - d[6];
  o[0] = d[0] + u + w + y * 32.f;
  o[1] = v + x + x + z * 16.f;
  o[2] = u + w * 4.f + y * 8.f;
  o[3] = v + x * 8.f + z * 4.f;
  o[4] = u + w * 16.f + y + y;
  o[5] = v + x * 32.f + z + d[7];
}

// ---- input transform: NCHW -> V[T][C][N*tiles]; one thread per (n, c, tile) ------------
template <int TILE>
__global__ void __launch_bounds__(256) wino_input_kernel(const WinoParams p) {
  constexpr int IN = TILE + 2;
  mb_grid_dep_launch();
  mb_grid_dep_wait();
  const int tiles = p.th * p.tw;
  const int64_t total = static_cast<int64_t>(p.N) * p.C * tiles;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int tile = static_cast<int>(tid % tiles);
  const int64_t r = tid / tiles;
  const int c = static_cast<int>(r % p.C);
  const int n = static_cast<int>(r / p.C);
  const int h0 = (tile / p.tw) * TILE - p.pad_t, w0 = (tile % p.tw) * TILE - p.pad_l;
  const float *ip = p.in + (static_cast<int64_t>(n) * p.C + c) * p.H * p.W;
  float d[IN][IN];
  // one address per patch row (the columns are constant offsets from it), the column tests made once
  bool col_ok[IN];
#pragma unroll
  for (int j = 0; j < IN; ++j) col_ok[j] = static_cast<unsigned>(w0 + j) < static_cast<unsigned>(p.W);
#pragma unroll
  for (int i = 0; i < IN; ++i) {
    const int h = h0 + i;
    const bool row_ok = static_cast<unsigned>(h) < static_cast<unsigned>(p.H);
    const float *rowp = ip + ((row_ok ? h : 0) * p.W + w0);
#pragma unroll
    for (int j = 0; j < IN; ++j) d[i][j] = (row_ok && col_ok[j]) ? __ldg(rowp + j) : 0.f;
  }
  const int64_t ncols = static_cast<int64_t>(p.N) * tiles;
  float *op = p.V + static_cast<int64_t>(c) * ncols + static_cast<int64_t>(n) * tiles + tile;
  if (TILE == 2) {
    const float *x = &d[0][0];
    float s[16];
    s[0] = (x[0] - x[8]) - (x[2] - x[10]);
    s[1] = (x[1] - x[9]) + (x[2] - x[10]);
    s[2] = (x[2] - x[10]) - (x[1] - x[9]);
    s[3] = (x[1] - x[9]) - (x[3] - x[11]);
    s[4] = (x[4] + x[8]) - (x[6] + x[10]);
    s[5] = (x[5] + x[9]) + (x[6] + x[10]);
    s[6] = (x[6] + x[10]) - (x[5] + x[9]);
    s[7] = (x[5] + x[9]) - (x[7] + x[11]);
    s[8] = (x[8] - x[4]) - (x[10] - x[6]);
    s[9] = (x[9] - x[5]) + (x[10] - x[6]);
    s[10] = (x[10] - x[6]) - (x[9] - x[5]);
    s[11] = (x[9] - x[5]) - (x[11] - x[7]);
    s[12] = (x[4] - x[12]) - (x[6] - x[14]);
    s[13] = (x[5] - x[13]) + (x[6] - x[14]);
    s[14] = (x[6] - x[14]) - (x[5] - x[13]);
    s[15] = (x[5] - x[13]) - (x[7] - x[15]);
#pragma unroll
    for (int i = 0; i < 16; ++i) *at_pos(op, i, p.v_pos_bytes) = s[i];
  } else {
    float s[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) bt8(d[i], s[i]);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float col[8], o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) col[j] = s[j][i];
      bt8(col, o);
#pragma unroll
      for (int j = 0; j < 8; ++j) *at_pos(op, j * 8 + i, p.v_pos_bytes) = o[j];
    }
  }
}

// ---- output transform: M[T][O][N*tiles] -> NCHW (+ bias, activation) --------------------
template <int TILE>
__global__ void __launch_bounds__(256) wino_output_kernel(const WinoParams p) {
  mb_grid_dep_launch();
  mb_grid_dep_wait();
  const int tiles = p.th * p.tw;
  const int64_t total = static_cast<int64_t>(p.N) * p.O * tiles;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int tile = static_cast<int>(tid % tiles);
  const int64_t r = tid / tiles;
  const int m = static_cast<int>(r % p.O);
  const int n = static_cast<int>(r / p.O);
  const int64_t ncols = static_cast<int64_t>(p.N) * tiles;
  const float *ip = p.Mx + static_cast<int64_t>(m) * ncols + static_cast<int64_t>(n) * tiles + tile;
  const int h0 = (tile / p.tw) * TILE, w0 = (tile % p.tw) * TILE;
  float *op = p.out + (static_cast<int64_t>(n) * p.O + m) * p.Ho * p.Wo;
  const float bias = p.bias != nullptr ? p.bias[m] : 0.f;
  if (TILE == 2) {
    float d[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) d[i] = *at_pos(ip, i, p.m_pos_bytes);
    const float s0 = d[0] + d[1] + d[2], s1 = d[1] - d[2] - d[3];
    const float s2 = d[4] + d[5] + d[6], s3 = d[5] - d[6] - d[7];
    const float s4 = d[8] + d[9] + d[10], s5 = d[9] - d[10] - d[11];
    const float s6 = d[12] + d[13] + d[14], s7 = d[13] - d[14] - d[15];
    const float v[2][2] = {{s0 + s2 + s4, s1 + s3 + s5}, {s2 - s4 - s6, s3 - s5 - s7}};
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j)
        if (h0 + i < p.Ho && w0 + j < p.Wo) {
          float y = v[i][j];
          if (p.bias != nullptr) y += bias;
          op[(h0 + i) * p.Wo + w0 + j] = act_apply(y, p.act, p.max_limit, p.coef);
        }
  } else {
    float s[8][6];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float d[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) d[j] = *at_pos(ip, i * 8 + j, p.m_pos_bytes);
      at8(d, s[i]);
    }
#pragma unroll
    for (int i = 0; i < 6; ++i) {
      float col[8], o[6];
#pragma unroll
      for (int j = 0; j < 8; ++j) col[j] = s[j][i];
      at8(col, o);
#pragma unroll
      for (int j = 0; j < 6; ++j)
        if (h0 + j < p.Ho && w0 + i < p.Wo) {
          float y = o[j];
          if (p.bias != nullptr) y += bias;
          op[(h0 + j) * p.Wo + w0 + i] = act_apply(y, p.act, p.max_limit, p.coef);
        }
    }
  }
}

// ---- plane-at-a-time output transform ---------------------------------------------------------
// For F(6,3) on images of at most 256 tiles a block takes whole (image, channel) output planes
// through shared memory: the threads assemble their 6x6 tiles there and the block writes the
// planes, which are one contiguous run of the output, with 128-bit stores.  (The
// one-thread-per-tile kernel writes the output in 24-byte pieces.)  threads_per_plane is the
// tile count rounded up to a multiple of 32; a block holds 256 / threads_per_plane planes.
// The same idea for the INPUT transform (plane into shared memory, windows cut out of it) was
// measured 15 % slower than the kernel above, whose overlapping window reads hit L1, and for
// the small F(2,3) planes neither direction gains.
template <int TILE>
__global__ void __launch_bounds__(256)
wino_output_plane_kernel(const WinoParams p, int threads_per_plane, int planes_per_block) {
  extern __shared__ float sm[];  // [planes_per_block][Ho * Wo]
  mb_grid_dep_launch();
  mb_grid_dep_wait();
  const int tiles = p.th * p.tw;
  const int hw = p.Ho * p.Wo;
  const int64_t planes = static_cast<int64_t>(p.N) * p.O;
  const int64_t plane0 = static_cast<int64_t>(blockIdx.x) * planes_per_block;
  const int pl = threadIdx.x / threads_per_plane, tile = threadIdx.x - pl * threads_per_plane;
  const int64_t plane = plane0 + pl;
  if (pl < planes_per_block && plane < planes && tile < tiles) {
    const int n = static_cast<int>(plane / p.O), m = static_cast<int>(plane - static_cast<int64_t>(n) * p.O);
    const int64_t ncols = static_cast<int64_t>(p.N) * tiles;
    const float *ip = p.Mx + static_cast<int64_t>(m) * ncols + static_cast<int64_t>(n) * tiles + tile;
    const int ty = tile / p.tw, tx = tile - ty * p.tw;
    const int h0 = ty * TILE, w0 = tx * TILE;
    float *op = sm + pl * hw;
    const float bias = p.bias != nullptr ? p.bias[m] : 0.f;
    if (TILE == 2) {
      float d[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) d[i] = *at_pos(ip, i, p.m_pos_bytes);
      const float s0 = d[0] + d[1] + d[2], s1 = d[1] - d[2] - d[3];
      const float s2 = d[4] + d[5] + d[6], s3 = d[5] - d[6] - d[7];
      const float s4 = d[8] + d[9] + d[10], s5 = d[9] - d[10] - d[11];
      const float s6 = d[12] + d[13] + d[14], s7 = d[13] - d[14] - d[15];
      const float v[2][2] = {{s0 + s2 + s4, s1 + s3 + s5}, {s2 - s4 - s6, s3 - s5 - s7}};
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
          if (h0 + i < p.Ho && w0 + j < p.Wo) {
            float y = v[i][j];
            if (p.bias != nullptr) y += bias;
            op[(h0 + i) * p.Wo + w0 + j] = act_apply(y, p.act, p.max_limit, p.coef);
          }
    } else {
      float s[8][6];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float d[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) d[j] = *at_pos(ip, i * 8 + j, p.m_pos_bytes);
        at8(d, s[i]);
      }
#pragma unroll
      for (int i = 0; i < 6; ++i) {
        float col[8], o[6];
#pragma unroll
        for (int j = 0; j < 8; ++j) col[j] = s[j][i];
        at8(col, o);
#pragma unroll
        for (int j = 0; j < 6; ++j)
          if (h0 + j < p.Ho && w0 + i < p.Wo) {
            float y = o[j];
            if (p.bias != nullptr) y += bias;
            op[(h0 + j) * p.Wo + w0 + i] = act_apply(y, p.act, p.max_limit, p.coef);
          }
      }
    }
  }
  __syncthreads();
  // the block's planes are one contiguous run of the output
  const int64_t count = min(static_cast<int64_t>(planes_per_block), planes - plane0) * hw;
  float *dst = p.out + plane0 * hw;
  if (((reinterpret_cast<uintptr_t>(dst) | (static_cast<uintptr_t>(count) * 4)) & 15u) == 0) {
    const float4 *s4 = reinterpret_cast<const float4 *>(sm);
    float4 *d4 = reinterpret_cast<float4 *>(dst);
    for (int64_t i = threadIdx.x; i < count / 4; i += 256) d4[i] = s4[i];
  } else {
    for (int64_t i = threadIdx.x; i < count; i += 256) dst[i] = sm[i];
  }
}

int pick_tile(int64_t H, int64_t W, int tile_override) {
  if (tile_override == 2 || tile_override == 6) return tile_override;
  return (H > 16 && W > 16) ? 6 : 2;  // conv_2d_3x3_winograd.cc:41-46
}

}  // namespace

extern "C" {

int mb_winograd_transform_filter_f32(mb_context *ctx, const float *filter, float *transformed,
                                     int64_t C, int64_t O, int tile) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (C < 1 || O < 1 || (tile != 2 && tile != 6) || O * C >= (1ll << 31))
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_winograd_transform_filter_f32: bad argument");
  if (filter == nullptr || transformed == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_winograd_transform_filter_f32: null operand");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  const unsigned blocks = static_cast<unsigned>(ceil_div64(O * C, 256));
  if (tile == 2)
    wino_filter_2x2_kernel<<<blocks, 256, 0, ctx->stream>>>(filter, transformed, static_cast<int>(C),
                                                            static_cast<int>(O));
  else
    wino_filter_6x6_kernel<<<blocks, 256, 0, ctx->stream>>>(filter, transformed, static_cast<int>(C),
                                                            static_cast<int>(O));
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

int mb_conv3x3_winograd_f32_nchw(mb_context *ctx, const float *in, const float *filter,
                                 const float *transformed_filter, const float *bias, float *out,
                                 int64_t N, int64_t C, int64_t H, int64_t W, int64_t O, int pad_top,
                                 int pad_left, int64_t Ho, int64_t Wo, int activation,
                                 float max_limit, float coefficient, int tile_override) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (N < 0 || C < 1 || H < 1 || W < 1 || O < 1 || pad_top < 0 || pad_left < 0 || Ho < 0 || Wo < 0)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_conv3x3_winograd_f32_nchw: bad shape argument");
  if (!(activation == 0 || activation == 1 || activation == 2 || activation == 6))
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_conv3x3_winograd_f32_nchw: activation %d", activation);
  if (N == 0 || Ho == 0 || Wo == 0) return MB_SUCCESS;
  if (in == nullptr || out == nullptr || (filter == nullptr && transformed_filter == nullptr))
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_conv3x3_winograd_f32_nchw: null operand");
  if (Ho > H + 2 * 2 || Wo > W + 2 * 2)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_conv3x3_winograd_f32_nchw: output larger than a 3x3 stride-1 conv gives");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  const int tile = pick_tile(H, W, tile_override);
  const int T = (tile + 2) * (tile + 2);
  const int64_t th = ceil_div64(Ho, tile), tw = ceil_div64(Wo, tile), tiles = th * tw;
  const int64_t ncols = N * tiles;
  if (ncols >= (1ll << 31) || O * C >= (1ll << 31) || C * ncols >= (1ll << 30) || O * ncols >= (1ll << 30))
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_conv3x3_winograd_f32_nchw: tensor too large");
  size_t off = 0;
  const size_t off_u = off; off += transformed_filter == nullptr ? align_up(sizeof(float) * T * O * C, 256) : 0;
  const size_t off_v = off; off += align_up(sizeof(float) * T * C * ncols, 256);
  const size_t off_m = off; off += align_up(sizeof(float) * T * O * ncols, 256);
  uint8_t *scratch = nullptr;
  MB_RETURN_IF_ERROR(mb_scratch(ctx, off, reinterpret_cast<void **>(&scratch)));
  const float *U = transformed_filter;
  if (U == nullptr) {
    float *u = reinterpret_cast<float *>(scratch + off_u);
    MB_RETURN_IF_ERROR(mb_winograd_transform_filter_f32(ctx, filter, u, C, O, tile));
    U = u;
  }
  WinoParams p;
  p.in = in; p.bias = bias; p.out = out;
  p.V = reinterpret_cast<float *>(scratch + off_v);
  p.Mx = reinterpret_cast<const float *>(scratch + off_m);
  p.N = static_cast<int>(N); p.C = static_cast<int>(C); p.H = static_cast<int>(H); p.W = static_cast<int>(W);
  p.O = static_cast<int>(O); p.pad_t = pad_top; p.pad_l = pad_left;
  p.Ho = static_cast<int>(Ho); p.Wo = static_cast<int>(Wo);
  p.th = static_cast<int>(th); p.tw = static_cast<int>(tw);
  p.act = activation; p.max_limit = max_limit; p.coef = coefficient;
  p.v_pos_bytes = static_cast<uint32_t>(C * ncols * 4);
  p.m_pos_bytes = static_cast<uint32_t>(O * ncols * 4);
  {
    const unsigned blocks = static_cast<unsigned>(ceil_div64(N * C * tiles, 256));
    // (all three kernels of the convolution are chained: each waits for its predecessor where it
    // first touches global memory and lets its successor's CTAs set up meanwhile)
    if (tile == 2) MB_CUDA(ctx, mb_launch_chained(ctx, wino_input_kernel<2>, dim3(blocks), dim3(256), 0, p));
    else MB_CUDA(ctx, mb_launch_chained(ctx, wino_input_kernel<6>, dim3(blocks), dim3(256), 0, p));
    MB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
  }
  // M_t [O x ncols] = U_t [O x C] * V_t [C x ncols] for t = 0 .. T-1
  MB_RETURN_IF_ERROR(mb_gemm_f32_strided(ctx, U, p.V, reinterpret_cast<float *>(scratch + off_m),
                                         nullptr, T, O, ncols, C, C, 1, O * C, ncols, 1, C * ncols,
                                         ncols, 1, O * ncols, 0, 0.f, 0.f));
  // plane-at-a-time output transform: F(6,3), at most 256 tiles per image, planes within the
  // default 48 KB of dynamic shared memory
  const int threads_per_plane = static_cast<int>((tiles + 31) / 32 * 32);
  const int planes_per_block = threads_per_plane <= 256 ? 256 / threads_per_plane : 0;
  const size_t out_plane_bytes = sizeof(float) * Ho * Wo;
  const bool plane_out = ctx->wino_plane && tile == 6 && planes_per_block > 0 &&
                         planes_per_block * out_plane_bytes <= 48 * 1024;
  if (plane_out) {
    const unsigned blocks = static_cast<unsigned>(ceil_div64(N * O, planes_per_block));
    const size_t smem = planes_per_block * out_plane_bytes;
    MB_CUDA(ctx, mb_launch_chained(ctx, wino_output_plane_kernel<6>, dim3(blocks), dim3(256), smem, p, threads_per_plane,
                                   planes_per_block));
    MB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
  } else {
    const unsigned blocks = static_cast<unsigned>(ceil_div64(N * O * tiles, 256));
    if (tile == 2) MB_CUDA(ctx, mb_launch_chained(ctx, wino_output_kernel<2>, dim3(blocks), dim3(256), 0, p));
    else MB_CUDA(ctx, mb_launch_chained(ctx, wino_output_kernel<6>, dim3(blocks), dim3(256), 0, p));
    MB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
  }
  return MB_SUCCESS;
}

}  // extern "C"
