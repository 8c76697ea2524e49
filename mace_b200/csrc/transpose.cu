// Batched 2-D transposes: the NHWC <-> NCHW conversions at the edge of a network.
//
// Reference behaviour: ops::Transpose as BaseFlow::TransposeInput / TransposeOutput call it
// with the permutations {0, 3, 1, 2} and {0, 2, 3, 1} (mace/core/flow/base_flow.cc:131-204,
// mace/flows/cpu/cpu_ref_flow.cc:81-101), and the Transpose operator for the same
// permutations and for {1, 0} (mace/ops/transpose.cc).  Per image both are the transpose of
// a [rows x cols] matrix: NHWC -> NCHW has rows = H * W, cols = C; NCHW -> NHWC the opposite.
// Pure data movement, so every output byte equals an input byte.
#include "common.cuh"

namespace {

// out[b][c][r] = in[b][r][c] through a 32 x 33 shared-memory tile: reads and writes both run
// along the contiguous dimension of their matrix.  Tiles of all images are spread over the
// grid by a grid-stride loop, so one launch covers any batch.
template <typename T>
__global__ void __launch_bounds__(256)
transpose_batched_kernel(const T *__restrict__ in, T *__restrict__ out, int64_t batch, int rows, int cols) {
  __shared__ T tile[32][33];
  const int tiles_c = (cols + 31) >> 5, tiles_r = (rows + 31) >> 5;
  const int64_t per_image = static_cast<int64_t>(tiles_c) * tiles_r;
  const int64_t total = per_image * batch;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int64_t b = t / per_image;
    const int rem = static_cast<int>(t - b * per_image);
    const int r0 = (rem / tiles_c) << 5, c0 = (rem % tiles_c) << 5;
    const T *src = in + b * static_cast<int64_t>(rows) * cols;
    T *dst = out + b * static_cast<int64_t>(rows) * cols;
#pragma unroll
    for (int i = ty; i < 32; i += 8)
      if (r0 + i < rows && c0 + tx < cols) tile[i][tx] = __ldg(src + static_cast<int64_t>(r0 + i) * cols + c0 + tx);
    __syncthreads();
#pragma unroll
    for (int i = ty; i < 32; i += 8)
      if (c0 + i < cols && r0 + tx < rows) dst[static_cast<int64_t>(c0 + i) * rows + r0 + tx] = tile[tx][i];
    __syncthreads();
  }
}

template <typename T>
int launch_transpose(mb_context *ctx, const void *in, void *out, int64_t batch, int64_t rows, int64_t cols) {
  const int64_t tiles = batch * ceil_div64(rows, 32) * ceil_div64(cols, 32);
  const int64_t grid = std::min<int64_t>(tiles, 16ll * ctx->num_sms);
  transpose_batched_kernel<T><<<static_cast<unsigned>(grid), 256, 0, ctx->stream>>>(
      static_cast<const T *>(in), static_cast<T *>(out), batch, static_cast<int>(rows), static_cast<int>(cols));
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches += 1;
  return MB_SUCCESS;
}

}  // namespace

extern "C" int mb_transpose2d_batched(mb_context *ctx, const void *in, void *out, int64_t batch, int64_t rows,
                                      int64_t cols, int elem_bytes) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (batch < 0 || rows < 0 || cols < 0 || rows > INT32_MAX || cols > INT32_MAX)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_transpose2d_batched: bad extents");
  if (elem_bytes != 1 && elem_bytes != 4)
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_transpose2d_batched: elements of 1 or 4 bytes only");
  if (batch == 0 || rows == 0 || cols == 0) return MB_SUCCESS;
  if (in == nullptr || out == nullptr || in == out)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_transpose2d_batched: null or aliased buffers");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  if (elem_bytes == 4) return launch_transpose<uint32_t>(ctx, in, out, batch, rows, cols);
  return launch_transpose<uint8_t>(ctx, in, out, batch, rows, cols);
}
