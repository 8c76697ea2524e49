// fp32 GEMM on the Blackwell tensor cores (tcgen05.mma kind::tf32) with split-operand error
// compensation, bias and activation fused into the epilogue.
//
// What it serves: the batched product of the Winograd convolution
// (arm::Conv2dK3x3Winograd, mace/ops/arm/base/conv_2d_3x3_winograd.cc:147-170, which calls
// arm::Gemm per image), the 1x1 convolution (arm::Conv2dK1x1,
// mace/ops/arm/base/conv_2d_1x1.cc:61-68) and MatMul/Gemm (mace/ops/arm/base/gemm.cc:520-683)
// in the layout all three share:
//     C[b][n][m] = act(bias[n] + sum_k X[b][k][m] * W[b][n][k])
// X is [K x Mdim] with m contiguous (an activation matrix: channels x pixels), W is
// [Ndim x K] with k contiguous (a filter matrix: output channels x channels), C is
// [Ndim x Mdim] with m contiguous (output channels x pixels).  The long pixel dimension is
// the tensor core's M (TMEM lanes), so that a warp's stores of one output channel cover 32
// consecutive pixels.
//
// Precision.  kind::tf32 reads only the upper 19 bits of each fp32 operand.  Every operand
// tile is therefore split in shared memory into hi = x with the low 13 mantissa bits
// cleared and lo = x - hi (exact), and each K step issues three MMAs,
//     hi*hi + lo*hi + hi*lo,
// into the fp32 accumulator; the dropped lo*lo term is below 2^-22 of the product, so the
// result matches an fp32 FMA loop to a few ulps (tests bound it at 1e-4 of the output range).
//
// Structure (one persistent CTA per SM, 448 threads):
//   warp 0        TMA producer: X as four [32 k x 32 m] boxes and W as one [BN x 32 k] box per
//                 stage, 128-byte swizzle, mbarrier ring
//   warp 1        MMA issuer (one thread)
//   warps 2..5    split: hi/lo tiles of the landed stage, then release it to the MMA warp
//   warps 6..13   epilogue: two sets of four warps (one per TMEM lane quarter), each on half
//                 of the tile's columns: tcgen05.ld, bias, activation, coalesced stores
// Every wait is bounded; on a timeout the kernel records a status word, lets outstanding
// copies land, frees its TMEM and returns.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

using namespace sm100;

constexpr int FBM = 128;       // pixels (m) per tile == TMEM lanes
constexpr int FKB = 32;        // k per pipeline stage (32 fp32 = one 128-byte swizzle row of W)
constexpr int FUMMA_K = 8;     // k per tcgen05.mma for tf32
constexpr int F_SPLIT_WARPS = 4;
constexpr int F_EPI_WARPS = 8;
constexpr int F_FIRST_EPI_WARP = 2 + F_SPLIT_WARPS;
constexpr int F_THREADS = (2 + F_SPLIT_WARPS + F_EPI_WARPS) * 32;
constexpr long long F_WAIT_BUDGET = 1ll << 31;

struct F32TcParams {
  int64_t Mdim, Ndim, K, batch;
  int tiles_m, tiles_n, k_blocks;
  int step_m, step_n, step_b;
  int x_batched, w_batched;
  const float *bias;  // per n, or null
  int act;
  float max_limit, coef;
  float *C;
  int64_t c_row_stride, c_batch_stride;  // elements between consecutive n / batch entries
  int c_tma;  // C rows are 16-byte aligned: written by TMA stores from shared memory
  int *status;
  long long *timeline;  // null, or clock stamps of CTA 0 (profiling aid): 5 per tile from slot 32
};

#ifdef MB_TC_TIMELINE
#define MBF_STAMP_TILE(tile, k)                                                     \
  do {                                                                              \
    if (p.timeline != nullptr && blockIdx.x == 0 && (tile) < 16)                    \
      p.timeline[32 + (tile) * 5 + (k)] = clock64();                                \
  } while (0)
#else
#define MBF_STAMP_TILE(tile, k) do { (void)(tile); } while (0)
#endif

template <int BN>
struct F32Cfg {
  static constexpr int X_BYTES = FBM * FKB * 4;   // 16 KB: four [32 k][32 m] sub-tiles of 4 KB
  static constexpr int W_BYTES = BN * FKB * 4;    // [BN n][32 k]
  static constexpr int HI_BYTES = X_BYTES + W_BYTES;
  static constexpr int STAGE_BYTES = 2 * HI_BYTES;  // hi tiles, then lo tiles
  // epilogue staging for the TMA stores: two buffers of 16 channels x 32 pixels per warp
  static constexpr int STAGING_BYTES = F_EPI_WARPS * 2 * 16 * 128;
  static constexpr int RING_BUDGET = 208 * 1024 - STAGING_BYTES;
  static constexpr int STAGES = RING_BUDGET / STAGE_BYTES > 6 ? 6 : RING_BUDGET / STAGE_BYTES;
  static_assert(STAGES >= 2, "pipeline needs two stages");
  static constexpr int NUM_ACC = 2;
  static constexpr int TMEM_COLS = 512;
  static constexpr int BAR_BYTES = 512;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 + BAR_BYTES;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

struct FTileIter {
  int tm, tn, b;
  __device__ __forceinline__ FTileIter(const F32TcParams &p) {
    const unsigned t = blockIdx.x;
    tm = t % p.tiles_m;
    const unsigned q = t / p.tiles_m;
    tn = q % p.tiles_n;
    b = q / p.tiles_n;
  }
  __device__ __forceinline__ bool valid(const F32TcParams &p) const { return b < p.batch; }
  __device__ __forceinline__ void next(const F32TcParams &p) {
    tm += p.step_m;
    tn += p.step_n;
    b += p.step_b;
    if (tm >= p.tiles_m) { tm -= p.tiles_m; ++tn; }
    if (tn >= p.tiles_n) { tn -= p.tiles_n; ++b; }
  }
};

}  // namespace

namespace {

template <int BN>
__global__ void __launch_bounds__(F_THREADS, 1)
gemm_f32_tc_kernel(const __grid_constant__ CUtensorMap tmap_x,
                   const __grid_constant__ CUtensorMap tmap_w,
                   const __grid_constant__ CUtensorMap tmap_c, const F32TcParams p) {
  using Cfg = F32Cfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NUM_ACC = Cfg::NUM_ACC;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t *bars =
      reinterpret_cast<uint64_t *>(smem_aligned + STAGES * Cfg::STAGE_BYTES + Cfg::STAGING_BYTES);
  const uint32_t full_bar = smem_u32(bars);              // [STAGES] raw tiles landed
  const uint32_t split_bar = full_bar + 8 * STAGES;      // [STAGES] hi/lo tiles ready
  const uint32_t empty_bar = split_bar + 8 * STAGES;     // [STAGES] stage consumed
  const uint32_t tfull_bar = empty_bar + 8 * STAGES;     // [NUM_ACC] accumulator complete
  const uint32_t tempty_bar = tfull_bar + 8 * NUM_ACC;   // [NUM_ACC] accumulator drained
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * STAGES + 2 * NUM_ACC);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tmap_x);
    prefetch_tensormap(&tmap_w);
    if (p.c_tma) prefetch_tensormap(&tmap_c);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(split_bar + 8 * s, F_SPLIT_WARPS);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int b = 0; b < NUM_ACC; ++b) {
      mbar_init(tfull_bar + 8 * b, 1);
      mbar_init(tempty_bar + 8 * b, F_EPI_WARPS);
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

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int local = 0;
#ifdef MB_TC_TIMELINE
    if (lane == 0 && p.timeline != nullptr && blockIdx.x == 0) p.timeline[0] = clock64();
#endif
    for (FTileIter it(p); ok && it.valid(p); it.next(p), ++local) {
      const int xb = p.x_batched ? it.b : 0, wb = p.w_batched ? it.b : 0;
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait_warp(empty_bar + 8 * stage, phase ^ 1, abort_flag, F_WAIT_BUDGET)) {
          *abort_flag = 1;
          atomicCAS(p.status, 0, MB_DEV_TIMEOUT_PRODUCER);
          ok = false;
          break;
        }
        if (lane == 0) {
          const uint32_t fb = full_bar + 8 * stage;
          const uint32_t sx = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sw = sx + Cfg::X_BYTES;
          mbar_arrive_expect_tx(fb, Cfg::HI_BYTES);
#pragma unroll
          for (int j = 0; j < 4; ++j)  // four 32-pixel atoms of the 128-pixel tile
            tma_load_3d(sx + j * (FKB * 128), &tmap_x, fb, it.tm * FBM + j * 32, kb * FKB, xb);
          tma_load_3d(sw, &tmap_w, fb, kb * FKB, it.tn * BN, wb);
          if (kb == 0) MBF_STAMP_TILE(local, 0);
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc = make_idesc(/*c f32*/ 1, /*a tf32*/ 2, /*b tf32*/ 2, /*a mn*/ true,
                                          /*b mn*/ false, FBM, BN);
    int stage = 0;
    uint32_t phase = 0;
    int acc_buf = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    int local = 0;
    for (FTileIter it(p); ok && it.valid(p); it.next(p), ++local) {
      if (!mbar_wait_warp(tempty_bar + 8 * acc_buf, acc_phase ^ 1, abort_flag, F_WAIT_BUDGET)) {
        *abort_flag = 1;
        atomicCAS(p.status, 0, MB_DEV_TIMEOUT_MMA);
        break;
      }
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + acc_buf * BN;
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait_warp(split_bar + 8 * stage, phase, abort_flag, F_WAIT_BUDGET)) {
          *abort_flag = 1;
          atomicCAS(p.status, 0, MB_DEV_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (kb == p.k_blocks - 1 && lane == 0) MBF_STAMP_TILE(local, 1);
        const uint32_t sx = smem_base + stage * Cfg::STAGE_BYTES;
        const uint32_t sw = sx + Cfg::X_BYTES;
        const int64_t k_left = p.K - static_cast<int64_t>(kb) * FKB;
        const int ksteps = k_left >= FKB ? FKB / FUMMA_K
                                         : static_cast<int>((k_left + FUMMA_K - 1) / FUMMA_K);
        if (lane == 0) {
          for (int j = 0; j < ksteps; ++j) {
            // X (MN-major tf32): k-rows of 128 bytes (32 pixels) in the "128-byte swizzle
            // with 32-byte atoms" layout (descriptor layout type 1; the TMA map uses
            // SWIZZLE_128B_ATOM_32B), whose pattern repeats every 4 k-rows: 4-row groups are
            // 512 bytes apart (SBO), 32-pixel atoms FKB * 128 bytes apart (LBO); a K step of 8
            // covers two groups = 1024 bytes.  The plain 128-byte swizzle gives zeros here.
            // W (K-major): rows of 128 bytes (32 k), 8-row groups 1024 bytes apart; a K step
            // moves 32 bytes inside the swizzled row.
            const uint64_t x_hi = make_smem_desc(sx + j * 1024, FKB * 128, 512, 1);
            const uint64_t x_lo = make_smem_desc(sx + Cfg::HI_BYTES + j * 1024, FKB * 128, 512, 1);
            const uint64_t w_hi = make_smem_desc(sw + j * 32, 16, 1024, 2);
            const uint64_t w_lo = make_smem_desc(sw + Cfg::HI_BYTES + j * 32, 16, 1024, 2);
            mma_tf32_ss(d_tmem, x_lo, w_hi, idesc, (kb > 0 || j > 0) ? 1u : 0u);
            mma_tf32_ss(d_tmem, x_hi, w_lo, idesc, 1u);
            mma_tf32_ss(d_tmem, x_hi, w_hi, idesc, 1u);
          }
          mma_commit(empty_bar + 8 * stage);
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) break;
      if (lane == 0) {
        mma_commit(tfull_bar + 8 * acc_buf);
        MBF_STAMP_TILE(local, 2);
      }
      __syncwarp();
      if (++acc_buf == NUM_ACC) {
        acc_buf = 0;
        acc_phase ^= 1;
      }
    }
  } else if (warp < F_FIRST_EPI_WARP) {
    // ---------------- split: hi / lo tiles ----------------
    const int t = (warp - 2) * 32 + lane;  // 0..127
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (FTileIter it(p); ok && it.valid(p); it.next(p)) {
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait_warp(full_bar + 8 * stage, phase, abort_flag, F_WAIT_BUDGET)) {
          *abort_flag = 1;
          atomicCAS(p.status, 0, MB_DEV_TIMEOUT_EPILOGUE);
          ok = false;
          break;
        }
        uint4 *hi = reinterpret_cast<uint4 *>(smem_aligned + stage * Cfg::STAGE_BYTES);
        uint4 *lo = reinterpret_cast<uint4 *>(smem_aligned + stage * Cfg::STAGE_BYTES + Cfg::HI_BYTES);
        // the split is element-wise, so the swizzled placement does not matter
#pragma unroll 4
        for (int i = t; i < Cfg::HI_BYTES / 16; i += F_SPLIT_WARPS * 32) {
          const uint4 v = hi[i];
          uint4 h, l;
          h.x = v.x & 0xffffe000u; h.y = v.y & 0xffffe000u;
          h.z = v.z & 0xffffe000u; h.w = v.w & 0xffffe000u;
          l.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(h.x));
          l.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(h.y));
          l.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(h.z));
          l.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(h.w));
          hi[i] = h;
          lo[i] = l;
        }
        fence_proxy_async();  // the MMA reads these tiles through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(split_bar + 8 * stage);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;
    const int set = (warp - F_FIRST_EPI_WARP) >> 2;  // 0, 1: which half of the columns
    constexpr int CHUNKS = BN / 16 / 2;              // 16-column chunks per warp
    // The activation as clamp + negative-slope term, with the choice made once: a branch
    // per value costs more than the arithmetic (few warps are there to hide its latency).
    //   NOOP: [-inf, inf], 0   RELU: [0, inf], 0   RELUX: [0, max_limit], 0   LEAKYRELU: [0, inf], coef
    const float act_lo = p.act == 0 ? -INFINITY : 0.f;
    const float act_hi = p.act == 2 ? p.max_limit : INFINITY;
    const float act_slope = p.act == 6 ? p.coef : 0.f;
    const bool leaky = p.act == 6;
    const float *bias = p.bias;
    const int64_t Ndim = p.Ndim;
    const int c_tma = p.c_tma;
    int acc_buf = 0;
    uint32_t acc_phase = 0;
    int local = 0;
    for (FTileIter it(p); it.valid(p); it.next(p), ++local) {
      if (!mbar_wait_warp(tfull_bar + 8 * acc_buf, acc_phase, abort_flag, F_WAIT_BUDGET)) {
        *abort_flag = 1;
        atomicCAS(p.status, 0, MB_DEV_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after_sync();
      if (warp == F_FIRST_EPI_WARP && lane == 0) MBF_STAMP_TILE(local, 3);
      const int64_t m = static_cast<int64_t>(it.tm) * FBM + quarter * 32 + lane;
      const bool m_ok = m < p.Mdim;
      float *c = p.C + it.b * p.c_batch_stride + m;
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc_buf * BN +
                             set * (BN / 2);
      const int64_t n_first = static_cast<int64_t>(it.tn) * BN + set * (BN / 2);
      uint32_t r[2][16];
      tmem_ld_32x32b_x16(tbase, r[0]);
      // staging: [buffer][channel j][pixel lane]; a lane's 16 writes of a chunk go to 16
      // different rows, the warp's write of one row covers all 32 banks
      float *stage_f = reinterpret_cast<float *>(smem_aligned + STAGES * Cfg::STAGE_BYTES +
                                                 (warp - F_FIRST_EPI_WARP) * (2 * 16 * 128));
      const int m0 = it.tm * FBM + quarter * 32;
#pragma unroll
      for (int i = 0; i < CHUNKS; ++i) {
        tmem_ld_wait_x16(r[i & 1]);
        if (i + 1 < CHUNKS) tmem_ld_32x32b_x16(tbase + (i + 1) * 16, r[(i + 1) & 1]);
        if (i == CHUNKS - 1) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar + 8 * acc_buf);
        }
        const int64_t n0 = n_first + i * 16;
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float bj = (bias != nullptr && n0 + j < Ndim) ? __ldg(bias + n0 + j) : 0.f;
          const float x = __uint_as_float(r[i & 1][j]) + bj;
          const float neg = leaky ? fminf(x, 0.f) * act_slope : 0.f;
          v[j] = fminf(fmaxf(x, act_lo), act_hi) + neg;
        }
        if (c_tma) {
          float *buf = stage_f + (i & 1) * (16 * 32);
          // the store that last used this buffer (two chunks ago) must have read it
          if (lane == 0) bulk_wait_group_read<1>();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 16; ++j) buf[j * 32 + lane] = v[j];
          fence_proxy_async();
          __syncwarp();
          if (lane == 0 && n0 < p.Ndim && m0 < p.Mdim) {
            tma_store_3d(&tmap_c, smem_u32(buf), m0, static_cast<int>(n0), it.b);
            bulk_commit_group();
          }
        } else if (m_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (n0 + j < p.Ndim) c[(n0 + j) * p.c_row_stride] = v[j];
        }
      }
      if (warp == F_FIRST_EPI_WARP && lane == 0) MBF_STAMP_TILE(local, 4);
      if (++acc_buf == NUM_ACC) {
        acc_buf = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) bulk_wait_group<0>();  // staging must outlive the stores' reads
    __syncwarp();
  }

  __syncthreads();
#ifdef MB_TC_TIMELINE
  if (threadIdx.x == 0 && p.timeline != nullptr && blockIdx.x == 0) p.timeline[15] = clock64();
#endif
  if (*abort_flag != 0) {
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

// 3-D fp32 tensor map: dims {inner, rows, batch} in elements, 128-byte swizzle, zero fill.
// Every stride must be a multiple of 16 bytes, that of a batch dimension of extent 1 too:
// callers pass row stride x rows there.
int make_map_f32(mb_context *ctx, CUtensorMap *map, const void *base, uint64_t inner, uint64_t rows,
                 uint64_t batch, uint64_t row_stride_elems, uint64_t batch_stride_elems,
                 uint32_t box_inner, uint32_t box_rows,
                 CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  const cuuint64_t dims[3] = {inner, rows, batch};
  const cuuint64_t strides[2] = {row_stride_elems * 4, batch_stride_elems * 4};
  const cuuint32_t box[3] = {box_inner, box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(base), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return mb_fail(ctx, MB_RUNTIME_ERROR, "cuTensorMapEncodeTiled (fp32) failed (%d)", static_cast<int>(r));
  return MB_SUCCESS;
}

template <int BN>
int launch_f32(mb_context *ctx, const CUtensorMap &tx, const CUtensorMap &tw, const CUtensorMap &tc,
               F32TcParams &p, int cfg_bit) {
  using Cfg = F32Cfg<BN>;
  auto kern = gemm_f32_tc_kernel<BN>;
  if (!(ctx->func_attr_mask & (1ull << cfg_bit))) {
    MB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    ctx->func_attr_mask |= (1ull << cfg_bit);
  }
  const int64_t total = p.batch * p.tiles_m * p.tiles_n;
  const int grid = static_cast<int>(total < ctx->num_sms ? total : ctx->num_sms);
  p.step_m = grid % p.tiles_m;
  p.step_n = (grid / p.tiles_m) % p.tiles_n;
  p.step_b = (grid / p.tiles_m) / p.tiles_n;
  kern<<<grid, F_THREADS, Cfg::SMEM_BYTES, ctx->stream>>>(tx, tw, tc, p);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  ctx->launches_tc++;
  return MB_SUCCESS;
}

}  // namespace

// Whether the tensor-core kernel can take C[b][n][m] = sum_k X[b][k][m] * W[b][n][k]: TMA needs
// 16-byte aligned bases and strides, i.e. row lengths that are multiples of four floats.
bool mb_gemm_f32_tc_supported(const mb_context *ctx, const float *X, const float *W, int64_t Mdim,
                              int64_t Ndim, int64_t K, int64_t x_row_stride, int64_t x_batch_stride,
                              int64_t w_row_stride, int64_t w_batch_stride) {
  if (ctx->encode_tiled == nullptr || !ctx->use_tensor_cores) return false;
  if (Mdim < 32 || Ndim < 1 || K < 1) return false;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W)) & 15u) return false;
  if ((x_row_stride % 4) || (x_batch_stride % 4) || (w_row_stride % 4) || (w_batch_stride % 4))
    return false;
  if (Mdim >= (1ll << 31) || Ndim >= (1ll << 31) || K >= (1ll << 31)) return false;
  return true;
}

int mb_gemm_f32_tc_launch(mb_context *ctx, const float *X, const float *W, const float *bias, float *C,
                          int64_t batch, int64_t Mdim, int64_t Ndim, int64_t K, int64_t x_row_stride,
                          int64_t x_batch_stride, int64_t w_row_stride, int64_t w_batch_stride,
                          int64_t c_row_stride, int64_t c_batch_stride, int act, float max_limit,
                          float coef) {
  const int BN = Ndim > 64 ? 128 : 64;
  F32TcParams p;
  p.Mdim = Mdim; p.Ndim = Ndim; p.K = K; p.batch = batch;
  p.tiles_m = static_cast<int>(ceil_div64(Mdim, FBM));
  p.tiles_n = static_cast<int>(ceil_div64(Ndim, BN));
  p.k_blocks = static_cast<int>(ceil_div64(K, FKB));
  p.x_batched = x_batch_stride != 0; p.w_batched = w_batch_stride != 0;
  p.bias = bias; p.act = act; p.max_limit = max_limit; p.coef = coef;
  p.C = C; p.c_row_stride = c_row_stride; p.c_batch_stride = c_batch_stride;
  p.status = ctx->dev_status;
  p.timeline = ctx->tc_timeline;
  CUtensorMap tx, tw;
  MB_RETURN_IF_ERROR(make_map_f32(ctx, &tx, X, Mdim, K, p.x_batched ? batch : 1, x_row_stride,
                                  p.x_batched ? x_batch_stride : x_row_stride * K, 32, FKB,
                                  CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B));
  MB_RETURN_IF_ERROR(make_map_f32(ctx, &tw, W, K, Ndim, p.w_batched ? batch : 1, w_row_stride,
                                  p.w_batched ? w_batch_stride : w_row_stride * Ndim, FKB, BN));
  CUtensorMap tc;
  p.c_tma = ((reinterpret_cast<uintptr_t>(C) & 15u) == 0 && c_row_stride % 4 == 0 &&
             c_batch_stride % 4 == 0 && Ndim >= 16) ? 1 : 0;
  if (p.c_tma) {
    MB_RETURN_IF_ERROR(make_map_f32(ctx, &tc, C, Mdim, Ndim, batch, c_row_stride,
                                    batch > 1 ? c_batch_stride : c_row_stride * Ndim, 32, 16,
                                    CU_TENSOR_MAP_SWIZZLE_NONE));
  } else {
    memset(&tc, 0, sizeof(tc));
  }
  if (BN == 128) return launch_f32<128>(ctx, tx, tw, tc, p, 41);
  return launch_f32<64>(ctx, tx, tw, tc, p, 42);
}
