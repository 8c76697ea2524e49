// uint8 x uint8 -> int32 GEMM on the Blackwell tensor cores (tcgen05.mma
// kind::i8) with the whole gemmlowp output pipeline fused into the epilogue.
//
// What it replaces: gemmlowp::GemmWithOutputPipeline as called by MACE's
// quantized MatMul and Conv2D (mace/ops/matmul.cc:283-301, :369-385;
// mace/ops/conv_2d.cc:301-315) with the output stages of
// mace/ops/common/gemmlowp_util.h:37-74.
//
// Formulation.  The tensor core multiplies the raw bytes:
//   raw[m,n] = sum_k A[m,k] * B[k,n]                      (exact in int32)
// and the epilogue applies the zero-point correction
//   acc = raw - zp_b * rowsum_A[m] - zp_a * colsum_B[n] + K * zp_a * zp_b
// then + bias, fixed-point requantization, + zp_c, clamp, store.
//
// Structure (one persistent CTA per SM, 320 threads):
//   warp 0      TMA producer: 128-byte-swizzled tiles of A and B into a
//               multi-stage shared-memory ring (mbarrier full/empty pairs)
//   warp 1      MMA issuer: one thread issues tcgen05.mma 128 x BN x 32 steps
//               into one of two TMEM accumulator buffers
//   warps 2..9  epilogue: tcgen05.ld the finished accumulator, correct,
//               requantize and store while the next tile is being multiplied
// Every wait is bounded; on a timeout the kernel records a status word, lets
// outstanding copies land, frees its TMEM and returns.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128;        // rows of A per tile == TMEM lanes
constexpr int BK = 128;        // bytes of K per pipeline stage (one swizzle row)
constexpr int UMMA_K = 32;     // K per tcgen05.mma for 8-bit operands
constexpr int EPI_WARPS = 8;
constexpr int NUM_THREADS = (2 + EPI_WARPS) * 32;
constexpr long long WAIT_BUDGET = 1ll << 31;  // ~1 s of SM clocks per wait
constexpr uint32_t SWIZZLE_128B = 2;

struct TcParams {
  int64_t M, N, K, batch;
  int tiles_m, tiles_n, k_blocks;
  int64_t total_tiles;
  const uint32_t *sum_a;  // [batch or 1][M]; may be null when zp_b == 0
  const uint32_t *sum_b;  // [batch or 1][N]; may be null when zp_a == 0
  int64_t sum_a_bstride, sum_b_bstride;
  int a_batched, b_batched;
  const int32_t *bias;
  int bias_per_row;
  int32_t zp_a, zp_b, kzz;
  mb_requant_params rq;
  void *C;
  int out_is_int32;
  int vec_store_ok;  // rows of C are 16-byte aligned
  int *status;
};

template <int BN, bool B_MN>
struct TileCfg {
  static constexpr int A_BYTES = BM * BK;
  static constexpr int B_BYTES = B_MN ? ((BN + 127) / 128) * 128 * BK : BN * BK;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (200 * 1024) / STAGE_BYTES > 8 ? 8 : (200 * 1024) / STAGE_BYTES;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_u8_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b, const TcParams p) {
  using Cfg = TileCfg<BN, B_MN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  // barrier block after the tile ring
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_aligned + STAGES * Cfg::STAGE_BYTES);
  const uint32_t full_bar = smem_u32(bars);                  // [STAGES]
  const uint32_t empty_bar = full_bar + 8 * STAGES;          // [STAGES]
  const uint32_t tfull_bar = empty_bar + 8 * STAGES;         // [2]
  const uint32_t tempty_bar = tfull_bar + 16;                // [2]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar + 8 * b, 1);
      mbar_init(tempty_bar + 8 * b, EPI_WARPS);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_batch = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
        const int b = static_cast<int>(tile / tiles_per_batch);
        const int rem = static_cast<int>(tile % tiles_per_batch);
        const int tm = rem % p.tiles_m, tn = rem / p.tiles_m;
        const int ab = p.a_batched ? b : 0, bb = p.b_batched ? b : 0;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1, abort_flag, WAIT_BUDGET)) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, MB_DEV_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          const uint32_t fb = full_bar + 8 * stage;
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + Cfg::A_BYTES;
          mbar_arrive_expect_tx(fb, Cfg::STAGE_BYTES);
          if (A_MN) {
            tma_load_3d(sa, &tmap_a, fb, tm * BM, kb * BK, ab);
          } else {
            tma_load_3d(sa, &tmap_a, fb, kb * BK, tm * BM, ab);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < (BN + 127) / 128; ++j)
              tma_load_3d(sb + j * 128 * BK, &tmap_b, fb, tn * BN + j * 128, kb * BK, bb);
          } else {
            tma_load_3d(sb, &tmap_b, fb, kb * BK, tn * BN, bb);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(/*c s32*/ 2, /*a u8*/ 0, /*b u8*/ 0, A_MN, B_MN, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int acc_buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar + 8 * acc_buf, acc_phase ^ 1, abort_flag, WAIT_BUDGET)) {
          *abort_flag = 1;
          atomicCAS(p.status, 0, MB_DEV_TIMEOUT_MMA);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc_buf * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, WAIT_BUDGET)) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, MB_DEV_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + Cfg::A_BYTES;
          const int64_t k_left = p.K - static_cast<int64_t>(kb) * BK;
          const int ksteps = k_left >= BK ? BK / UMMA_K
                                          : static_cast<int>((k_left + UMMA_K - 1) / UMMA_K);
#pragma unroll 4
          for (int j = 0; j < ksteps; ++j) {
            // K-major tile: rows of 128 bytes, 8-row groups 1024 bytes apart;
            // a K step moves 32 bytes inside the swizzled row.
            // MN-major tile: k-rows of 128 bytes (128 elements of M or N),
            // 8-k-row groups 1024 bytes apart, 128-element atoms 16 KB apart;
            // a K step moves 32 k-rows = 4096 bytes.
            const uint64_t a_desc =
                A_MN ? make_smem_desc(sa + j * UMMA_K * 128, 128 * BK, 1024, SWIZZLE_128B)
                     : make_smem_desc(sa + j * UMMA_K, 16, 1024, SWIZZLE_128B);
            const uint64_t b_desc =
                B_MN ? make_smem_desc(sb + j * UMMA_K * 128, 128 * BK, 1024, SWIZZLE_128B)
                     : make_smem_desc(sb + j * UMMA_K, 16, 1024, SWIZZLE_128B);
            mma_i8_ss(d_tmem, a_desc, b_desc, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          mma_commit(empty_bar + 8 * stage);  // frees the stage when the MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        mma_commit(tfull_bar + 8 * acc_buf);  // accumulator complete
        acc_buf ^= 1;
        if (acc_buf == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int ew = warp - 2;
    const int quarter = warp & 3;          // TMEM lanes [32*quarter, +32) are this warp's
    const int col_half = ew >> 2;          // two warps share a lane quarter, split columns
    constexpr int CHUNKS = BN / 32;
    constexpr int CHUNKS_PER_WARP = CHUNKS >= 2 ? CHUNKS / 2 : 1;
    int acc_buf = 0;
    uint32_t acc_phase = 0;
    for (int64_t tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
      const int b = static_cast<int>(tile / tiles_per_batch);
      const int rem = static_cast<int>(tile % tiles_per_batch);
      const int tm = rem % p.tiles_m, tn = rem / p.tiles_m;
      if (!mbar_wait(tfull_bar + 8 * acc_buf, acc_phase, abort_flag, WAIT_BUDGET)) {
        *abort_flag = 1;
        atomicCAS(p.status, 0, MB_DEV_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after_sync();
      const int64_t m = static_cast<int64_t>(tm) * BM + quarter * 32 + lane;
      const bool row_ok = m < p.M;
      int32_t row_term = 0;
      if (row_ok) {
        if (p.sum_a != nullptr)
          row_term -= p.zp_b * static_cast<int32_t>(
                                   p.sum_a[(p.a_batched ? b : 0) * p.sum_a_bstride + m]);
        if (p.bias != nullptr && p.bias_per_row) row_term += p.bias[m];
      }
      const uint32_t *sum_b = p.sum_b ? p.sum_b + (p.b_batched ? b : 0) * p.sum_b_bstride : nullptr;
      uint8_t *c8 = static_cast<uint8_t *>(p.C) + (static_cast<int64_t>(b) * p.M + m) * p.N;
      int32_t *c32 = static_cast<int32_t *>(p.C) + (static_cast<int64_t>(b) * p.M + m) * p.N;
      if (CHUNKS >= 2 || col_half == 0) {
#pragma unroll 1
        for (int ci = 0; ci < CHUNKS_PER_WARP; ++ci) {
          const int chunk = col_half * CHUNKS_PER_WARP + ci;
          const int64_t n0 = static_cast<int64_t>(tn) * BN + chunk * 32;
          if (n0 >= p.N) break;  // uniform across the warp
          uint32_t r[32];
          const uint32_t taddr =
              tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc_buf * BN + chunk * 32;
          tmem_ld_32x32b_x32(taddr, r);
          // column term of this lane's column, broadcast by shuffle below
          int32_t col_term = p.kzz;
          const int64_t nl = n0 + lane;
          if (nl < p.N) {
            if (sum_b != nullptr) col_term -= p.zp_a * static_cast<int32_t>(sum_b[nl]);
            if (p.bias != nullptr && !p.bias_per_row) col_term += p.bias[nl];
          }
          tmem_ld_wait();
          if (p.out_is_int32) {
            int32_t v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = static_cast<int32_t>(r[j]) + row_term + __shfl_sync(0xffffffffu, col_term, j);
            if (row_ok) {
              if (p.vec_store_ok && n0 + 32 <= p.N) {
                uint4 *dst = reinterpret_cast<uint4 *>(c32 + n0);
#pragma unroll
                for (int q = 0; q < 8; ++q)
                  dst[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (n0 + j < p.N) c32[n0 + j] = v[j];
              }
            }
          } else {
            uint32_t packed[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              uint32_t w = 0;
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int j = 4 * q + e;
                const int32_t acc = static_cast<int32_t>(r[j]) + row_term +
                                    __shfl_sync(0xffffffffu, col_term, j);
                w |= mb_requant_fast(acc, p.rq) << (8 * e);
              }
              packed[q] = w;
            }
            if (row_ok) {
              if (p.vec_store_ok && n0 + 32 <= p.N) {
                uint4 *dst = reinterpret_cast<uint4 *>(c8 + n0);
                dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (n0 + j < p.N) c8[n0 + j] = static_cast<uint8_t>(packed[j >> 2] >> (8 * (j & 3)));
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar + 8 * acc_buf);
      acc_buf ^= 1;
      if (acc_buf == 0) acc_phase ^= 1;
    }
  }

  __syncthreads();
  if (*abort_flag != 0) {
    // Give copies and MMAs that are still in flight time to land before the
    // shared memory and TMEM they target go away (bounded: about 2 ms).
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 3-D uint8 tensor map: dims {inner, rows, batch}, 128-byte swizzle.
int make_map_u8(mb_context *ctx, CUtensorMap *map, const void *base, uint64_t inner,
                uint64_t rows, uint64_t batch, uint64_t batch_stride_bytes, uint32_t box_inner,
                uint32_t box_rows) {
  const cuuint64_t dims[3] = {inner, rows, batch};
  const cuuint64_t strides[2] = {inner, batch_stride_bytes};
  const cuuint32_t box[3] = {box_inner, box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return mb_fail(ctx, MB_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
  return MB_SUCCESS;
}

template <int BN, bool A_MN, bool B_MN>
int launch_cfg(mb_context *ctx, const CUtensorMap &ta, const CUtensorMap &tb, TcParams &p) {
  using Cfg = TileCfg<BN, B_MN>;
  auto kern = gemm_u8_tc_kernel<BN, A_MN, B_MN>;
  // The opt-in shared-memory limit is a per-device function attribute; set it
  // once per context.
  constexpr int cfg_id = (BN == 256 ? 0 : BN == 128 ? 1 : 2) * 4 + (A_MN ? 2 : 0) + (B_MN ? 1 : 0);
  if (!(ctx->func_attr_mask & (1ull << cfg_id))) {
    MB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg::SMEM_BYTES));
    ctx->func_attr_mask |= (1ull << cfg_id);
  }
  const int grid = static_cast<int>(p.total_tiles < ctx->num_sms ? p.total_tiles : ctx->num_sms);
  kern<<<grid, NUM_THREADS, Cfg::SMEM_BYTES, ctx->stream>>>(ta, tb, p);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  ctx->launches_tc++;
  return MB_SUCCESS;
}

}  // namespace

// Whether the tensor-core path can take this problem: TMA needs 16-byte
// aligned bases and row strides, and raw byte products must not wrap int32.
bool mb_gemm_u8_tc_supported(const mb_context *ctx, const void *A, const void *B, int64_t M,
                             int64_t N, int64_t K, bool a_mn, bool b_mn, int a_batched,
                             int b_batched) {
  if (ctx->encode_tiled == nullptr) return false;
  if (M < 1 || N < 1 || K < 1) return false;
  if (K > 33000) return false;  // 255*255*K must stay below 2^31
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15u) return false;
  const int64_t a_inner = a_mn ? M : K, b_inner = b_mn ? N : K;
  if ((a_inner % 16) || (b_inner % 16)) return false;
  if (a_batched && ((M * K) % 16)) return false;
  if (b_batched && ((N * K) % 16)) return false;
  if (M > (1ll << 31) || N > (1ll << 31)) return false;
  return true;
}

// Launch the tensor-core GEMM.  A is [M x K] K-major (a_mn = false) or
// [K x M] MN-major; B^T is [N x K] K-major (b_mn = false) or B is [K x N]
// MN-major.  C is row-major M x N.  sum_a / sum_b are the per-row byte sums of
// the operands (may be null when the other zero point is 0).
int mb_gemm_u8_tc_launch(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                         const uint32_t *sum_a, const uint32_t *sum_b, const int32_t *bias,
                         void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N,
                         int64_t K, bool a_mn, bool b_mn, int a_batched, int b_batched,
                         int32_t zp_a, int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c,
                         int bias_per_row) {
  int BN = 256;
  {
    // Prefer the widest tile that still gives every SM a tile.
    const int64_t tm = ceil_div64(M, BM);
    const int widths[3] = {256, 128, 64};
    BN = 64;
    for (int w : widths) {
      if (N >= w && batch * tm * ceil_div64(N, w) >= ctx->num_sms) {
        BN = w;
        break;
      }
    }
    if (N <= 64) BN = 64;
    else if (N <= 128 && BN > 128) BN = 128;
  }
  TcParams p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.tiles_m = static_cast<int>(ceil_div64(M, BM));
  p.tiles_n = static_cast<int>(ceil_div64(N, BN));
  p.k_blocks = static_cast<int>(ceil_div64(K, BK));
  p.total_tiles = batch * p.tiles_m * p.tiles_n;
  p.sum_a = sum_a; p.sum_b = sum_b;
  p.sum_a_bstride = M; p.sum_b_bstride = N;
  p.a_batched = a_batched; p.b_batched = b_batched;
  p.bias = bias; p.bias_per_row = bias_per_row;
  p.zp_a = zp_a; p.zp_b = zp_b;
  p.rq = mb_make_requant(mult, shift, zp_c);
  p.kzz = static_cast<int32_t>(static_cast<uint32_t>(K) * static_cast<uint32_t>(zp_a) *
                               static_cast<uint32_t>(zp_b));
  p.C = C; p.out_is_int32 = out_is_int32;
  const uintptr_t cbase = reinterpret_cast<uintptr_t>(C);
  p.vec_store_ok = out_is_int32 ? ((cbase % 16 == 0) && (N % 4 == 0))
                                : ((cbase % 16 == 0) && (N % 16 == 0));
  p.status = ctx->dev_status;

  CUtensorMap ta, tb;
  const uint64_t nb_a = a_batched ? batch : 1, nb_b = b_batched ? batch : 1;
  if (a_mn) {
    MB_RETURN_IF_ERROR(make_map_u8(ctx, &ta, A, M, K, nb_a, M * K, 128, BK));
  } else {
    MB_RETURN_IF_ERROR(make_map_u8(ctx, &ta, A, K, M, nb_a, M * K, BK, BM));
  }
  if (b_mn) {
    MB_RETURN_IF_ERROR(make_map_u8(ctx, &tb, B, N, K, nb_b, N * K, 128, BK));
  } else {
    MB_RETURN_IF_ERROR(make_map_u8(ctx, &tb, B, K, N, nb_b, N * K, BK, BN));
  }

#define MB_TC_DISPATCH(BN_)                                                         \
  if (a_mn) {                                                                       \
    if (b_mn) return launch_cfg<BN_, true, true>(ctx, ta, tb, p);                   \
    return launch_cfg<BN_, true, false>(ctx, ta, tb, p);                            \
  } else {                                                                          \
    if (b_mn) return launch_cfg<BN_, false, true>(ctx, ta, tb, p);                  \
    return launch_cfg<BN_, false, false>(ctx, ta, tb, p);                           \
  }
  if (BN == 256) { MB_TC_DISPATCH(256) }
  if (BN == 128) { MB_TC_DISPATCH(128) }
  MB_TC_DISPATCH(64)
#undef MB_TC_DISPATCH
}
