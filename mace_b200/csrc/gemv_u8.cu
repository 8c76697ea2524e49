// uint8 GEMV with the float requantization rule of MACE's Gemv delegators.
//
// Reference behaviour: arm::q8::Gemv<T>::Compute (mace/ops/arm/q8/gemv.cc:36-171):
//   ret = dot - sum_lhs * zp_rhs - sum_rhs * zp_lhs + K * zp_lhs * zp_rhs (+ bias[h])
//   uint8: Saturate<uint8_t>(roundf(ret * multiplier_float + zp_out))
// and ref::q8::Gemv<uint8_t> (mace/ops/ref/q8/gemv.cc:80-122), which omits
// zp_out.  The product and the sum are rounded separately (no fused
// multiply-add), as the C++ expression is written.
//
// The kernel is bandwidth-bound: one warp streams one row of the matrix with
// 128-bit loads and integer dot-product instructions.  When the matrix is shared by all
// batch entries (the FullyConnected case) the warp keeps its row and loops over the vectors.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

struct GemvParams {
  const uint8_t *lhs, *rhs;
  const int32_t *bias;
  void *out;
  int64_t batch, rows, K;
  int lhs_batched, rhs_batched, out_is_int32, add_zp_out;
  int32_t zp_lhs, zp_rhs, zp_out;
  float multiplier;
  int batch_chunk;
};

// One warp per matrix row.  The first 4 KB of the row are requested before anything else (8
// independent 128-bit loads per lane in flight); the vector's bytes and their sum are the
// same for every row of the block, so they are staged in shared memory once per block and
// batch entry.  A matrix shared by the batch is loaded once and kept in registers.
template <bool VEC>
__global__ void __launch_bounds__(256) gemv_u8_kernel(const GemvParams p) {
  extern __shared__ uint4 xs[];  // VEC: the vector, K / 16 words
  __shared__ uint32_t sum_r_sm;
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const bool row_ok = row < p.rows;
  // blockIdx.y walks the batch: one entry per block when every entry has its
  // own matrix, otherwise a chunk of entries that share the warp's matrix row.
  const int64_t b_begin = p.lhs_batched ? blockIdx.y : static_cast<int64_t>(blockIdx.y) * p.batch_chunk;
  const int64_t b_end = p.lhs_batched ? b_begin + 1 : min(p.batch, b_begin + p.batch_chunk);
  uint4 l[8];
  for (int64_t b = b_begin; b < b_end; ++b) {
    const uint8_t *lp = p.lhs + (p.lhs_batched ? b * p.rows * p.K : 0) + (row_ok ? row : 0) * p.K;
    const uint8_t *rp = p.rhs + (p.rhs_batched ? b * p.K : 0);
    uint32_t dot = 0, sum_l = 0, sum_r = 0;
    if (VEC) {
      const int nvec = static_cast<int>(p.K >> 4);
      const uint4 *l4 = reinterpret_cast<const uint4 *>(lp);
      const uint4 *r4 = reinterpret_cast<const uint4 *>(rp);
      // the matrix row first: its loads are the long-latency ones
      const int pre = min(8, (nvec - lane + 31) / 32);
      if (b == b_begin || p.lhs_batched) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (i < pre) l[i] = __ldg(l4 + lane + 32 * i);
      }
      __syncthreads();  // previous batch entry's readers are done with xs
      uint32_t part = 0;
      for (int i = threadIdx.x; i < nvec; i += 256) {
        const uint4 r = __ldg(r4 + i);
        xs[i] = r;
        part = __dp4a(r.x, 0x01010101u, part);
        part = __dp4a(r.y, 0x01010101u, part);
        part = __dp4a(r.z, 0x01010101u, part);
        part = __dp4a(r.w, 0x01010101u, part);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      if (threadIdx.x == 0) sum_r_sm = 0;
      __syncthreads();
      if (lane == 0) atomicAdd(&sum_r_sm, part);
      __syncthreads();
      sum_r = sum_r_sm;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i < pre) {
          const uint4 r = xs[lane + 32 * i];
          dot = __dp4a(l[i].x, r.x, dot); dot = __dp4a(l[i].y, r.y, dot);
          dot = __dp4a(l[i].z, r.z, dot); dot = __dp4a(l[i].w, r.w, dot);
          sum_l = __dp4a(l[i].x, 0x01010101u, sum_l); sum_l = __dp4a(l[i].y, 0x01010101u, sum_l);
          sum_l = __dp4a(l[i].z, 0x01010101u, sum_l); sum_l = __dp4a(l[i].w, 0x01010101u, sum_l);
        }
      }
#pragma unroll 4
      for (int i = lane + 256; i < nvec; i += 32) {
        const uint4 lv = __ldg(l4 + i);
        const uint4 r = xs[i];
        dot = __dp4a(lv.x, r.x, dot); dot = __dp4a(lv.y, r.y, dot);
        dot = __dp4a(lv.z, r.z, dot); dot = __dp4a(lv.w, r.w, dot);
        sum_l = __dp4a(lv.x, 0x01010101u, sum_l); sum_l = __dp4a(lv.y, 0x01010101u, sum_l);
        sum_l = __dp4a(lv.z, 0x01010101u, sum_l); sum_l = __dp4a(lv.w, 0x01010101u, sum_l);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        dot += __shfl_xor_sync(0xffffffffu, dot, o);
        sum_l += __shfl_xor_sync(0xffffffffu, sum_l, o);
      }
    } else {
      for (int64_t i = lane; i < p.K; i += 32) {
        const uint32_t l = lp[i], r = rp[i];
        dot += l * r;
        sum_l += l;
        sum_r += r;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        dot += __shfl_xor_sync(0xffffffffu, dot, o);
        sum_l += __shfl_xor_sync(0xffffffffu, sum_l, o);
        sum_r += __shfl_xor_sync(0xffffffffu, sum_r, o);
      }
    }
    if (lane == 0 && row_ok) {
      const uint32_t zero_point_dot = static_cast<uint32_t>(
          static_cast<int64_t>(p.zp_lhs) * p.zp_rhs * p.K);
      int32_t ret = static_cast<int32_t>(dot - sum_l * static_cast<uint32_t>(p.zp_rhs) -
                                         sum_r * static_cast<uint32_t>(p.zp_lhs) + zero_point_dot);
      if (p.bias != nullptr) ret += p.bias[row];
      const int64_t idx = b * p.rows + row;
      if (p.out_is_int32) {
        static_cast<int32_t *>(p.out)[idx] = ret;
      } else {
        float v = __fmul_rn(static_cast<float>(ret), p.multiplier);
        if (p.add_zp_out) v = __fadd_rn(v, static_cast<float>(p.zp_out));
        static_cast<uint8_t *>(p.out)[idx] = static_cast<uint8_t>(mb_saturate_round_u8(v));
      }
    }
  }
}

// ---- one vector against a large matrix: the matrix streams through shared memory ---------------
//
// The matrix is read exactly once and nothing else moves, so the kernel is a copy engine with
// a dot product behind it.  A persistent grid (two CTAs per SM) divides the rows into
// contiguous, equally long runs, one per CTA, so that every SM streams the same number of
// bytes.  Inside a CTA each of the 8 warps owns a private ring of ST_DEPTH slots of ST_CHUNK
// bytes; lane 0 asks for a row chunk with one untiled bulk copy (cp.async.bulk) that signals
// the slot's mbarrier, the warp multiplies the landed chunk with the vector (staged in shared
// memory once per CTA) and lane 0 refills the slot: up to 8 x ST_DEPTH x 4 KB are in flight per
// CTA with no thread holding registers for them, and no warp waits for another.
// Bounded waits: a wait that runs out sets the context's status word and the warp stops.
constexpr int ST_CHUNK_MAX = 4096;   // bytes of a matrix row per bulk copy (template CHUNK: 4096, or 2048 for chains)
constexpr int ST_DEPTH = 3;      // slots per warp
constexpr int ST_WARPS = 8;
constexpr long long ST_WAIT_BUDGET = 1ll << 31;

struct GemvStreamParams {
  const uint8_t *lhs, *rhs;
  const int32_t *bias;
  void *out;
  int64_t rows, K;
  int out_is_int32, add_zp_out;
  int32_t zp_lhs, zp_rhs, zp_out;
  float multiplier;
  int lhs_const;   // the matrix is not written by work ahead in the stream (a weight)
  int *status;
};

template <int ST_CHUNK>
__global__ void __launch_bounds__(ST_WARPS * 32) gemv_u8_stream_kernel(const GemvStreamParams p) {
  extern __shared__ __align__(128) uint8_t st_smem[];
  // [ST_WARPS][ST_DEPTH][ST_CHUNK] ring, then the vector (K bytes), then the barriers
  uint8_t *ring = st_smem;
  uint4 *xs = reinterpret_cast<uint4 *>(st_smem + ST_WARPS * ST_DEPTH * ST_CHUNK);
  uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(xs) + p.K);
  __shared__ uint32_t sum_r_sm;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  mb_grid_dep_launch();
  if (threadIdx.x == 0) {
    for (int i = 0; i < ST_WARPS * ST_DEPTH; ++i) sm100::mbar_init(sm100::smem_u32(bars + i), 1);
    sum_r_sm = 0;
    abort_flag = 0;
    sm100::fence_barrier_init();
  }
  __syncthreads();
  // this CTA's rows: an equal share of the matrix, contiguous
  const int64_t r_begin = p.rows * blockIdx.x / gridDim.x;
  const int64_t r_end = p.rows * (blockIdx.x + 1) / gridDim.x;
  const int chunks_per_row = static_cast<int>((p.K + ST_CHUNK - 1) / ST_CHUNK);
  // this warp's units: (row, chunk) pairs of rows r_begin + warp, + 8, ...
  const int64_t my_rows = r_begin + warp < r_end ? (r_end - r_begin - warp + ST_WARPS - 1) / ST_WARPS : 0;
  const int64_t units = my_rows * chunks_per_row;
  uint8_t *my_ring = ring + warp * (ST_DEPTH * ST_CHUNK);
  const uint32_t my_bar = sm100::smem_u32(bars + warp * ST_DEPTH);
  auto issue = [&](int64_t u) {  // lane 0 only
    const int64_t row = r_begin + warp + (u / chunks_per_row) * ST_WARPS;
    const int c = static_cast<int>(u % chunks_per_row);
    const uint32_t bytes = static_cast<uint32_t>(min(static_cast<int64_t>(ST_CHUNK), p.K - static_cast<int64_t>(c) * ST_CHUNK));
    const int slot = static_cast<int>(u % ST_DEPTH);
    sm100::mbar_arrive_expect_tx(my_bar + 8 * slot, bytes);
    sm100::bulk_load_1d(sm100::smem_u32(my_ring + slot * ST_CHUNK), p.lhs + row * p.K + static_cast<int64_t>(c) * ST_CHUNK,
                        bytes, my_bar + 8 * slot);
  };
  // A weight matrix may be fetched before the work ahead in the stream has finished: the ring's
  // first fill then overlaps the previous kernel's tail (or all of it, for a chain of such
  // products).  The vector and the output are touched only after the wait.
  if (p.lhs_const && lane == 0)
    for (int64_t u = 0; u < units && u < ST_DEPTH; ++u) issue(u);
  mb_grid_dep_wait();  // from here on every operand may be read
  if (!p.lhs_const && lane == 0)
    for (int64_t u = 0; u < units && u < ST_DEPTH; ++u) issue(u);
  // the vector and its byte sum, once per CTA, while the first chunks are on their way
  {
    const int nvec = static_cast<int>(p.K >> 4);
    const uint4 *r4 = reinterpret_cast<const uint4 *>(p.rhs);
    uint32_t part = 0;
    for (int i = threadIdx.x; i < nvec; i += ST_WARPS * 32) {
      const uint4 r = __ldg(r4 + i);
      xs[i] = r;
      part = __dp4a(r.x, 0x01010101u, part);
      part = __dp4a(r.y, 0x01010101u, part);
      part = __dp4a(r.z, 0x01010101u, part);
      part = __dp4a(r.w, 0x01010101u, part);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) atomicAdd(&sum_r_sm, part);
  }
  __syncthreads();
  const uint32_t sum_r = sum_r_sm;
  const uint32_t zero_point_dot = static_cast<uint32_t>(static_cast<int64_t>(p.zp_lhs) * p.zp_rhs * p.K);
  uint32_t dot = 0, sum_l = 0;
  for (int64_t u = 0; u < units; ++u) {
    const int slot = static_cast<int>(u % ST_DEPTH);
    const uint32_t parity = static_cast<uint32_t>((u / ST_DEPTH) & 1);
    if (!sm100::mbar_wait_warp(my_bar + 8 * slot, parity, &abort_flag, ST_WAIT_BUDGET)) {
      abort_flag = 1;
      if (lane == 0) atomicCAS(p.status, 0, MB_DEV_TIMEOUT_PRODUCER);
      break;
    }
    const int c = static_cast<int>(u % chunks_per_row);
    const int vec0 = c * (ST_CHUNK / 16);
    const int nv = static_cast<int>(min(static_cast<int64_t>(ST_CHUNK / 16), (p.K >> 4) - vec0));
    const uint4 *w4 = reinterpret_cast<const uint4 *>(my_ring + slot * ST_CHUNK);
#pragma unroll 4
    for (int i = lane; i < nv; i += 32) {
      const uint4 lv = w4[i];
      const uint4 r = xs[vec0 + i];
      dot = __dp4a(lv.x, r.x, dot); dot = __dp4a(lv.y, r.y, dot);
      dot = __dp4a(lv.z, r.z, dot); dot = __dp4a(lv.w, r.w, dot);
      sum_l = __dp4a(lv.x, 0x01010101u, sum_l); sum_l = __dp4a(lv.y, 0x01010101u, sum_l);
      sum_l = __dp4a(lv.z, 0x01010101u, sum_l); sum_l = __dp4a(lv.w, 0x01010101u, sum_l);
    }
    // the slot has been read (the values are in registers): refill it
    __syncwarp();
    if (lane == 0 && u + ST_DEPTH < units) {
      sm100::fence_proxy_async();
      issue(u + ST_DEPTH);
    }
    if (c == chunks_per_row - 1) {  // end of a row
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        dot += __shfl_xor_sync(0xffffffffu, dot, o);
        sum_l += __shfl_xor_sync(0xffffffffu, sum_l, o);
      }
      if (lane == 0) {
        const int64_t row = r_begin + warp + (u / chunks_per_row) * ST_WARPS;
        int32_t ret = static_cast<int32_t>(dot - sum_l * static_cast<uint32_t>(p.zp_rhs) -
                                           sum_r * static_cast<uint32_t>(p.zp_lhs) + zero_point_dot);
        if (p.bias != nullptr) ret += p.bias[row];
        if (p.out_is_int32) {
          static_cast<int32_t *>(p.out)[row] = ret;
        } else {
          float v = __fmul_rn(static_cast<float>(ret), p.multiplier);
          if (p.add_zp_out) v = __fadd_rn(v, static_cast<float>(p.zp_out));
          static_cast<uint8_t *>(p.out)[row] = static_cast<uint8_t>(mb_saturate_round_u8(v));
        }
      }
      dot = 0;
      sum_l = 0;
    }
  }
  // a warp that gave up may still have copies in flight into this CTA's shared memory: let
  // them land before the CTA ends (bounded)
  if (abort_flag != 0)
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
}

}  // namespace

bool mb_gemm_u8_tc_supported(const mb_context *ctx, const void *A, const void *B, int64_t M,
                             int64_t N, int64_t K, bool a_mn, bool b_mn, int a_batched,
                             int b_batched);
int mb_gemm_u8_tc_launch_float_rule(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                                    const int32_t *bias, void *C, int out_is_int32, int64_t M,
                                    int64_t N, int64_t K, int32_t zp_a, int32_t zp_b, float mult_f,
                                    int32_t zp_c, int add_zp);

extern "C" int mb_gemv_u8(mb_context *ctx, const uint8_t *lhs, const uint8_t *rhs,
                          const int32_t *bias, void *out, int out_is_int32, int64_t batch,
                          int64_t rows, int64_t K, int lhs_batched, int rhs_batched,
                          int32_t zp_lhs, int32_t zp_rhs, float multiplier, int32_t zp_out,
                          int add_zp_out) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (batch < 0 || rows < 0 || K < 0)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_gemv_u8: negative dimension");
  if (batch == 0 || rows == 0) return MB_SUCCESS;
  if (lhs == nullptr || rhs == nullptr || out == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_gemv_u8: null operand");
  if (lhs_batched && batch > 65535)
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_gemv_u8: batch > 65535 with a batched matrix");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  // Many vectors against one matrix (FullyConnected on a batch) is a GEMM
  // out[batch x rows] = rhs[batch x K] * lhs[rows x K]^T: the tensor-core kernel with the float
  // requantization rule in its epilogue reads the matrix once instead of once per vector.
  if (!lhs_batched && rhs_batched && batch >= 16 && K % 16 == 0 && K <= 1024 && ctx->use_tensor_cores &&
      mb_gemm_u8_tc_supported(ctx, rhs, lhs, batch, rows, K, false, false, 0, 0)) {
    ctx->gemm_b_const = ctx->gemv_lhs_const;  // the matrix is the GEMM's B
    const int st = mb_gemm_u8_tc_launch_float_rule(ctx, rhs, lhs, bias, out, out_is_int32, batch, rows, K, zp_rhs,
                                           zp_lhs, multiplier, zp_out, add_zp_out);
    ctx->gemm_b_const = 0;
    return st;
  }
  // One vector against a large matrix: the streaming kernel (see gemv_u8_stream_kernel).
  if (batch == 1 && ctx->gemv_stream && K % 16 == 0 && K >= 256 && K <= 65536 && rows >= 2ll * ctx->num_sms &&
      ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) & 15u) == 0) {
    GemvStreamParams sp;
    sp.lhs = lhs; sp.rhs = rhs; sp.bias = bias; sp.out = out;
    sp.rows = rows; sp.K = K;
    sp.out_is_int32 = out_is_int32; sp.add_zp_out = add_zp_out;
    sp.zp_lhs = zp_lhs; sp.zp_rhs = zp_rhs; sp.zp_out = zp_out; sp.multiplier = multiplier;
    sp.status = ctx->dev_status;
    sp.lhs_const = ctx->gemv_lhs_const;
    // A constant matrix in a chain of such products: half-size chunks, so that FOUR CTAs fit an
    // SM -- two of this launch and two of the next one, whose first ring fill (issued ahead of
    // its dependency wait) is then under way while this launch still streams.  (option
    // gemv_const_one_per_sm = 1 instead leaves one of two full-size places to the successor.)
    const bool small_chunks = sp.lhs_const && ctx->gemv_chain_chunks && !ctx->gemv_const_one_per_sm;
    const int chunk = small_chunks ? 2048 : ST_CHUNK_MAX;
    const size_t smem = static_cast<size_t>(ST_WARPS) * ST_DEPTH * chunk + static_cast<size_t>(K) +
                        sizeof(uint64_t) * ST_WARPS * ST_DEPTH;
    const uint64_t attr_bit = small_chunks ? (1ull << 61) : (1ull << 62);
    if (!(ctx->func_attr_mask & attr_bit)) {
      if (small_chunks)
        MB_CUDA(ctx, cudaFuncSetAttribute(gemv_u8_stream_kernel<2048>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          ST_WARPS * ST_DEPTH * 2048 + 65536 + 8 * ST_WARPS * ST_DEPTH));
      else
        MB_CUDA(ctx, cudaFuncSetAttribute(gemv_u8_stream_kernel<ST_CHUNK_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          ST_WARPS * ST_DEPTH * ST_CHUNK_MAX + 65536 + 8 * ST_WARPS * ST_DEPTH));
      ctx->func_attr_mask |= attr_bit;
    }
    const int per_sm = (smem <= 110 * 1024 && !(sp.lhs_const && ctx->gemv_const_one_per_sm)) ? 2 : 1;
    const unsigned grid = static_cast<unsigned>(std::min<int64_t>(rows, static_cast<int64_t>(ctx->num_sms) * per_sm));
    if (small_chunks)
      MB_CUDA(ctx, mb_launch_chained(ctx, gemv_u8_stream_kernel<2048>, dim3(grid), dim3(ST_WARPS * 32), smem, sp));
    else
      MB_CUDA(ctx, mb_launch_chained(ctx, gemv_u8_stream_kernel<ST_CHUNK_MAX>, dim3(grid), dim3(ST_WARPS * 32), smem, sp));
    MB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
    return MB_SUCCESS;
  }
  GemvParams p;
  p.lhs = lhs; p.rhs = rhs; p.bias = bias; p.out = out;
  p.batch = batch; p.rows = rows; p.K = K;
  p.lhs_batched = lhs_batched; p.rhs_batched = rhs_batched;
  p.out_is_int32 = out_is_int32; p.add_zp_out = add_zp_out;
  p.zp_lhs = zp_lhs; p.zp_rhs = zp_rhs; p.zp_out = zp_out; p.multiplier = multiplier;
  const bool vec = (K % 16 == 0) && K > 0 && K <= 32768 &&
                   ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs)) & 15u) == 0;
  // a shared matrix: split the batch so that at least ~4 blocks per SM exist
  int64_t chunks = 1;
  if (!lhs_batched) {
    chunks = std::min<int64_t>(batch, std::max<int64_t>(1, (4ll * ctx->num_sms) / ceil_div64(rows, 8)));
    chunks = std::min<int64_t>(chunks, 65535);
  }
  p.batch_chunk = static_cast<int>(ceil_div64(batch, chunks));
  dim3 grid(static_cast<unsigned>(ceil_div64(rows, 8)),
            lhs_batched ? static_cast<unsigned>(batch)
                        : static_cast<unsigned>(ceil_div64(batch, p.batch_chunk)));
  if (vec) gemv_u8_kernel<true><<<grid, 256, static_cast<size_t>(K), ctx->stream>>>(p);
  else gemv_u8_kernel<false><<<grid, 256, 0, ctx->stream>>>(p);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}
