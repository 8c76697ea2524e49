// Byte sums of the GEMM operands for the zero-point correction
//   acc = raw - zp_b * rowsum_A[m] - zp_a * colsum_B[n] + K * zp_a * zp_b
// (what gemmlowp's packing stage computes on the fly for MACE's quantized MatMul,
// mace/ops/matmul.cc:283-301).  Both operands are summed by ONE launch: the first blocks take
// A, the rest B.  An operand stored with K contiguous ("K-major": [rows x K]) needs row sums --
// a warp per row.  One stored with M or N contiguous ([K x cols]) needs column sums: a block of
// eight warps covers 512 adjacent columns (a warp reads 512 contiguous bytes of a row with
// 128-bit loads) and one SLICE of the K rows, and writes the slice's sums as one partial row;
// the partial rows (at most 64) are added up by the GEMM where it reads the sums, so no block
// waits for another and nothing needs zeroing.  The kernel lets the GEMM behind it start at once
// (programmatic dependent launch): the GEMM's main loop does not need the sums, only its
// epilogue terms do, and those wait.
#include <algorithm>

#include "common.cuh"

namespace {

constexpr int SUM_WARPS = 8;

struct SumJob {
  const uint8_t *x;
  uint32_t *out;
  int kind;                  // 0: nothing, 1: row sums, 2: column sums
  int64_t nb;                // matrices
  int64_t rows, cols;        // kind 1: rows x cols(=K) per matrix; kind 2: K rows x cols
  int64_t pitch, mat_stride; // kind 1: bytes from row to row and from matrix to matrix
  int num_blocks;
  // column sums: out is [nb][slices][cols]
  int col_blocks, slices;
  int64_t rows_per_slice;
};

template <int WARPS>
__device__ __forceinline__ void row_sums(const SumJob &j, int block) {
  const int lane = threadIdx.x & 31;
  const int64_t total = j.nb * j.rows;
  const int64_t nvec = j.cols >> 4;
  for (int64_t row = static_cast<int64_t>(block) * WARPS + (threadIdx.x >> 5); row < total;
       row += static_cast<int64_t>(j.num_blocks) * WARPS) {
    const uint4 *p = reinterpret_cast<const uint4 *>(j.x + (row / j.rows) * j.mat_stride + (row % j.rows) * j.pitch);
    uint32_t s = 0;
#pragma unroll 8
    for (int64_t i = lane; i < nvec; i += 32) {
      const uint4 v = __ldg(p + i);
      s = __dp4a(v.x, 0x01010101u, s);
      s = __dp4a(v.y, 0x01010101u, s);
      s = __dp4a(v.z, 0x01010101u, s);
      s = __dp4a(v.w, 0x01010101u, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) j.out[row] = s;
  }
}

template <int WARPS>
__device__ __forceinline__ void col_sums(const SumJob &j, int block, uint32_t (*part)[32][17]) {
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int bx = block % j.col_blocks;
  const int rest = block / j.col_blocks;
  const int sy = rest % j.slices;
  const int64_t b = rest / j.slices;
  const int64_t c16 = static_cast<int64_t>(bx) * 32 + tx;  // 16-column group
  const bool active = c16 * 16 < j.cols;
  const int64_t r0 = static_cast<int64_t>(sy) * j.rows_per_slice;
  const int64_t r1 = min(j.rows, r0 + j.rows_per_slice);
  const uint8_t *base = j.x + b * j.rows * j.cols;
  uint32_t s[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) s[i] = 0;
  if (active) {
#pragma unroll 8
    for (int64_t r = r0 + ty; r < r1; r += WARPS) {
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(base + r * j.cols) + c16);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        s[4 * q + 0] = __dp4a(w[q], 0x00000001u, s[4 * q + 0]);
        s[4 * q + 1] = __dp4a(w[q], 0x00000100u, s[4 * q + 1]);
        s[4 * q + 2] = __dp4a(w[q], 0x00010000u, s[4 * q + 2]);
        s[4 * q + 3] = __dp4a(w[q], 0x01000000u, s[4 * q + 3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) part[ty][tx][i] = s[i];
  __syncthreads();
  // 512 columns: adjacent columns per thread, one partial row per slice
  uint32_t *dst = j.out + (b * j.slices + sy) * j.cols;
  for (int c = threadIdx.x; c < 512; c += WARPS * 32) {
    const int64_t col = static_cast<int64_t>(bx) * 512 + c;
    if (col >= j.cols) continue;
    uint32_t t = 0;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) t += part[w][c >> 4][c & 15];
    dst[col] = t;
  }
}

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) operand_sums_kernel(const SumJob a, const SumJob b) {
  __shared__ uint32_t part[WARPS][32][17];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int block = blockIdx.x;
  const SumJob &j = block < a.num_blocks ? a : b;
  const int local = block < a.num_blocks ? block : block - a.num_blocks;
  if (j.kind == 1) row_sums<WARPS>(j, local);
  else if (j.kind == 2) col_sums<WARPS>(j, local, part);
}

}  // namespace

// Partial rows the column sums of a [K x cols] operand are written as (1 for row sums).
int mb_operand_sums_slices(const mb_context *ctx, bool mn, int64_t nb, int64_t K, int64_t cols) {
  if (!mn) return 1;
  const int64_t col_blocks = ceil_div64(cols, 512);
  // enough blocks that the loads in flight (8 x 16 bytes per thread) cover the memory latency of
  // the whole GPU (measured on a 4096 x 4096 operand: 512 blocks of 256 threads read it in 8 us,
  // 256 blocks of 128 threads in 12 us), but, together with the row-sum blocks of the other
  // operand (two per SM), no more than the five blocks per SM that are resident at once: a
  // second, partial round of blocks cost the 4096^3 GEMM about a microsecond
  int64_t slices = ceil_div64(3ll * ctx->num_sms, col_blocks * nb);
  slices = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(slices, 64), ceil_div64(K, 32)));
  const int64_t rps = ceil_div64(K, slices);
  return static_cast<int>(ceil_div64(K, rps));
}

// Sums for A (row sums when K-major; partial column sums, mb_operand_sums_slices() rows of them,
// when a_mn) into sum_a and for B into sum_b; either output may be null (not needed).
// k_split > 1: single matrices (nb_a = nb_b = 1) whose depth is cut into k_split equal runs, each
// summed on its own as if it were a matrix of a batch (outputs [k_split][...]).
int mb_operand_sums_launch(mb_context *ctx, const uint8_t *A, bool a_mn, int64_t nb_a, int64_t M, uint32_t *sum_a,
                           const uint8_t *B, bool b_mn, int64_t nb_b, int64_t N, uint32_t *sum_b, int64_t K,
                           int k_split) {
  const int64_t k_full = K;
  if (k_split > 1) {
    K /= k_split;
    nb_a = nb_b = k_split;
  }
  auto make = [&](const uint8_t *x, bool mn, int64_t nb, int64_t extent, uint32_t *out) {
    SumJob j = {};
    if (out == nullptr) return j;
    j.x = x; j.out = out; j.nb = nb;
    if (!mn) {  // [extent x K], K contiguous
      j.kind = 1;
      j.rows = extent; j.cols = K;
      j.pitch = k_full;
      j.mat_stride = k_split > 1 ? K : extent * K;
      j.num_blocks = static_cast<int>(std::min<int64_t>(ceil_div64(nb * extent, SUM_WARPS),
                                                        static_cast<int64_t>(ctx->num_sms) * 2));
    } else {    // [K x extent] -> [slices][extent] partial rows
      j.kind = 2;
      j.rows = K; j.cols = extent;
      j.col_blocks = static_cast<int>(ceil_div64(extent, 512));
      j.slices = mb_operand_sums_slices(ctx, true, nb, K, extent);
      j.rows_per_slice = ceil_div64(K, j.slices);
      j.num_blocks = static_cast<int>(nb * j.col_blocks * j.slices);
    }
    return j;
  };
  const SumJob ja = make(A, a_mn, nb_a, M, sum_a);
  const SumJob jb = make(B, b_mn, nb_b, N, sum_b);
  const int64_t blocks = static_cast<int64_t>(ja.num_blocks) + jb.num_blocks;
  if (blocks == 0) return MB_SUCCESS;
  if (blocks > 0x7fffffffll) return mb_fail(ctx, MB_UNSUPPORTED, "operand sums: too many blocks");
  operand_sums_kernel<SUM_WARPS><<<static_cast<unsigned>(blocks), SUM_WARPS * 32, 0, ctx->stream>>>(ja, jb);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}
