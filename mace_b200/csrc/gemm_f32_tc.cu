// fp32 GEMM on the Blackwell tensor cores (tcgen05.mma kind::tf32) with split-operand error
// compensation, bias and activation fused into the epilogue.
//
// What it serves: the batched product of the Winograd convolution
// (arm::Conv2dK3x3Winograd, mace/ops/arm/base/conv_2d_3x3_winograd.cc:147-170, which calls
// arm::Gemm per image), the 1x1 convolution (arm::Conv2dK1x1,
// mace/ops/arm/base/conv_2d_1x1.cc:61-68), the im2col form of the general convolution and
// MatMul/Gemm (mace/ops/arm/base/gemm.cc:520-683) in the layout all of them share:
//     C[b][n][m] = act(bias[n] + sum_k X[b][k][m] * W[b][n][k] [+ R[b][n][m]])
// X is [K x Mdim] with m contiguous (an activation matrix: channels x pixels), W is
// [Ndim x K] with k contiguous (a filter matrix: output channels x channels), C is
// [Ndim x Mdim] with m contiguous (output channels x pixels).  The long pixel dimension is
// the tensor core's M (TMEM lanes), so that a warp's stores of one output channel cover 32
// consecutive pixels.
//
// Precision.  kind::tf32 reads only the upper 19 bits of each fp32 operand.  Every operand
// is therefore split into hi = x with the low 13 mantissa bits cleared and lo = x - hi
// (exact), and each K step issues three MMAs,
//     lo*hi + hi*lo + hi*hi,
// into the fp32 accumulator; the dropped lo*lo term is below 2^-22 of the product, so the
// result matches an fp32 FMA loop to a few ulps (tests bound it at 1e-4 of the output range).
//
// Where the split operands live.  The X operand (the MMA's A, 128 pixels = 128 TMEM lanes)
// goes to TENSOR MEMORY: a warp per lane quarter reads its pixels' 32 k-values of the landed
// tile from shared memory (one word per lane and k: conflict-free), splits them in registers
// and writes hi and lo with tcgen05.st into a ring of TMEM columns; the MMA takes A from
// there.  Only W (the MMA's B) is split in shared memory, in place.  Against splitting both
// operands in shared memory this halves the shared-memory bytes a K step moves (the MMA no
// longer reads A from it, and X is never written back) and shrinks a pipeline stage from
// 64 KB to 48 KB, so four stages fit instead of two; the loads then run far enough ahead to
// hide the memory latency, which had bounded the two-stage version.
//
// Structure (one persistent CTA per SM, 576 threads):
//   warp 0        TMA producer: X as one [32 k x 128 m] box (no swizzle) and W as one
//                 [BN x 32 k] box (128-byte swizzle) per stage, mbarrier ring
//   warp 1        MMA issuer (one thread): A from TMEM, B from shared memory
//   warps 2..5    X split: shared memory -> registers -> hi/lo in TMEM
//   warps 6..9    W split: hi/lo tiles in shared memory
//   warps 10..17  epilogue: two sets of four warps (one per TMEM lane quarter), each on half
//                 of the tile's columns: tcgen05.ld, bias, activation, TMA stores
// TMEM columns: two accumulators of BN columns, then STAGES x 64 columns of A (hi 32, lo 32).
// Every wait is bounded; on a timeout the kernel records a status word, lets outstanding
// copies land, frees its TMEM and returns.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

using namespace sm100;

constexpr int FBM = 128;       // pixels (m) per tile == TMEM lanes
constexpr int FKB = 32;        // k per pipeline stage (32 fp32 = one 128-byte swizzle row of W)
constexpr int FUMMA_K = 8;     // k per tcgen05.mma for tf32
constexpr int F_XSPLIT_WARPS = 4;   // one per TMEM lane quarter
constexpr int F_WSPLIT_WARPS = 4;
constexpr int F_SPLIT_WARPS = F_XSPLIT_WARPS + F_WSPLIT_WARPS;
constexpr int F_FIRST_WSPLIT_WARP = 2 + F_XSPLIT_WARPS;
constexpr int F_EPI_WARPS = 8;
constexpr int F_FIRST_EPI_WARP = 2 + F_SPLIT_WARPS;
constexpr int F_THREADS = (2 + F_SPLIT_WARPS + F_EPI_WARPS) * 32;
constexpr int F_A_COLS = 2 * FKB;   // TMEM columns of one stage's A operand: hi, then lo
constexpr long long F_WAIT_BUDGET = 1ll << 31;

struct F32TcParams {
  int64_t Mdim, Ndim, K, batch;
  int tiles_m, tiles_n, k_blocks;
  int step_m, step_n, step_b;
  int x_batched, w_batched;
  const float *bias;  // per n, or null
  const float *residual;  // null, or a tensor laid out like C that is added before the activation
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
// per K step of CTA 0 (first 64 steps): role 0 producer issue, 1 tile landed, 2 X split done,
// 3 MMA sees both splits, 4 MMAs issued, 5 W split done; slots from 128
#define MBF_STAMP_K(role, idx)                                                      \
  do {                                                                              \
    if (p.timeline != nullptr && blockIdx.x == 0 && (idx) < 64)                     \
      p.timeline[128 + (role) * 64 + (idx)] = clock64();                            \
  } while (0)
#else
#define MBF_STAMP_TILE(tile, k) do { (void)(tile); } while (0)
#define MBF_STAMP_K(role, idx) do { (void)(idx); } while (0)
#endif

template <int BN>
struct F32Cfg {
  static constexpr int X_BYTES = FBM * FKB * 4;   // 16 KB: [32 k][128 m]
  static constexpr int W_BYTES = BN * FKB * 4;    // [BN n][32 k]
  static constexpr int STAGE_BYTES = X_BYTES + 2 * W_BYTES;  // raw X, W hi (lands raw), W lo
  // epilogue staging for the TMA stores: two buffers of 16 channels x 128 pixels per warp set
  static constexpr int STAGING_BYTES = 2 * 2 * 16 * FBM * 4;
  static constexpr int BAR_BYTES = 512;
  static constexpr int RING_BUDGET = 227 * 1024 - STAGING_BYTES - 1024 - BAR_BYTES;
  static constexpr int NUM_ACC = 2;
  static constexpr int TMEM_COLS = 512;
  static constexpr int A_COL0 = NUM_ACC * BN;     // first TMEM column of the A ring
  static constexpr int MAX_TMEM_STAGES = (TMEM_COLS - A_COL0) / F_A_COLS;
  static constexpr int SMEM_STAGES = RING_BUDGET / STAGE_BYTES;
  static constexpr int STAGES = SMEM_STAGES < MAX_TMEM_STAGES ? SMEM_STAGES : MAX_TMEM_STAGES;
  static_assert(STAGES >= 2, "pipeline needs two stages");
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 + BAR_BYTES;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
  static_assert(3 * STAGES * 8 + 2 * NUM_ACC * 8 + 16 <= BAR_BYTES, "barrier area");
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

// EPI selects the epilogue's arithmetic: 1 = no bias, no residual, no activation (the Winograd
// products, whose output transform applies them): the accumulator is the result; 2 = bias,
// residual and a clamp (NOOP / RELU / RELUX); 0 = all of that plus the leaky term.
template <int BN, int EPI = 0>
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
  mb_grid_dep_launch();  // the kernel behind this one may start its own prologue

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
  // everything above touched only this CTA's shared and tensor memory; from here on the roles read
  // and write global memory, which the kernel in front of this one may still be producing
  mb_grid_dep_wait();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // One thread runs the role (see the MMA issuer); the other lanes wait at the warp barrier.
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      int kstep = 0;
#ifdef MB_TC_TIMELINE
      if (p.timeline != nullptr && blockIdx.x == 0) p.timeline[0] = clock64();
#endif
      for (FTileIter it(p); ok && it.valid(p); it.next(p), ++local) {
        const int xb = p.x_batched ? it.b : 0, wb = p.w_batched ? it.b : 0;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++kstep) {
          if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1, abort_flag, F_WAIT_BUDGET)) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, MB_DEV_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          const uint32_t fb = full_bar + 8 * stage;
          const uint32_t sx = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sw = sx + Cfg::X_BYTES;
          MBF_STAMP_K(0, kstep);
          mbar_arrive_expect_tx(fb, Cfg::X_BYTES + Cfg::W_BYTES);
          tma_load_3d(sx, &tmap_x, fb, it.tm * FBM, kb * FKB, xb);  // [32 k][128 m], 512-byte rows
          tma_load_3d(sw, &tmap_w, fb, kb * FKB, it.tn * BN, wb);
          if (kb == 0) MBF_STAMP_TILE(local, 0);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // One thread runs the whole role.  The tensor pipe queues only a few MMAs, so everything
    // between the last MMA of one K step and the first of the next (commit, barrier poll,
    // descriptor arithmetic) has to fit into the time those queued MMAs take to execute, or
    // the pipe idles: the descriptors are one add per K step, the common four-step case is
    // unrolled, and nothing in the loop is warp-collective.
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(/*c f32*/ 1, /*a tf32*/ 2, /*b tf32*/ 2, /*a mn*/ false,
                                            /*b mn*/ false, FBM, BN);
      // W (K-major): rows of 128 bytes (32 k), 8-row groups 1024 bytes apart; a K step of 8
      // moves 32 bytes inside the swizzled row (+2 in the descriptor's address field).
      const uint64_t wdesc = make_smem_desc(0, 16, 1024, 2);
      const int last_ksteps =
          static_cast<int>((p.K - static_cast<int64_t>(p.k_blocks - 1) * FKB + FUMMA_K - 1) / FUMMA_K);
      int stage = 0;
      uint32_t phase = 0;
      int acc_buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      int local = 0;
      int kstep = 0;
      for (FTileIter it(p); ok && it.valid(p); it.next(p), ++local) {
        if (!mbar_wait(tempty_bar + 8 * acc_buf, acc_phase ^ 1, abort_flag, F_WAIT_BUDGET)) {
          *abort_flag = 1;
          atomicCAS(p.status, 0, MB_DEV_TIMEOUT_MMA);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc_buf * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++kstep) {
          if (!mbar_wait(split_bar + 8 * stage, phase, abort_flag, F_WAIT_BUDGET)) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, MB_DEV_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (kb == p.k_blocks - 1) MBF_STAMP_TILE(local, 1);
          MBF_STAMP_K(3, kstep);
          const uint32_t sw = smem_base + stage * Cfg::STAGE_BYTES + Cfg::X_BYTES;
          // A (TMEM): lane = pixel, one column per k; a K step of 8 is 8 columns; hi in the
          // first 32 columns of the stage's slot, lo in the next 32.
          const uint32_t a_hi = tmem_base + Cfg::A_COL0 + stage * F_A_COLS, a_lo = a_hi + FKB;
          const uint64_t w_hi = wdesc | static_cast<uint64_t>((sw >> 4) & 0x3FFFu);
          const uint64_t w_lo = wdesc | static_cast<uint64_t>(((sw + Cfg::W_BYTES) >> 4) & 0x3FFFu);
          if (kb + 1 < p.k_blocks || last_ksteps == FKB / FUMMA_K) {
#pragma unroll
            for (int j = 0; j < FKB / FUMMA_K; ++j) {
              mma_tf32_ts(d_tmem, a_lo + j * FUMMA_K, w_hi + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
              mma_tf32_ts(d_tmem, a_hi + j * FUMMA_K, w_lo + 2 * j, idesc, 1u);
              mma_tf32_ts(d_tmem, a_hi + j * FUMMA_K, w_hi + 2 * j, idesc, 1u);
            }
          } else {
            for (int j = 0; j < last_ksteps; ++j) {
              mma_tf32_ts(d_tmem, a_lo + j * FUMMA_K, w_hi + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
              mma_tf32_ts(d_tmem, a_hi + j * FUMMA_K, w_lo + 2 * j, idesc, 1u);
              mma_tf32_ts(d_tmem, a_hi + j * FUMMA_K, w_hi + 2 * j, idesc, 1u);
            }
          }
          mma_commit(empty_bar + 8 * stage);
          MBF_STAMP_K(4, kstep);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        mma_commit(tfull_bar + 8 * acc_buf);
        MBF_STAMP_TILE(local, 2);
        if (++acc_buf == NUM_ACC) {
          acc_buf = 0;
          acc_phase ^= 1;
        }
      }
    }
    __syncwarp();
  } else if (warp < F_FIRST_WSPLIT_WARP) {
    // ---------------- X split: shared memory -> hi / lo in tensor memory ----------------
    const int quarter = warp & 3;  // the TMEM lanes this warp may touch: 32 * (warp % 4) ...
    const uint32_t a_lane = static_cast<uint32_t>(quarter * 32) << 16;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int kstep = 0;
    for (FTileIter it(p); ok && it.valid(p); it.next(p)) {
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait_warp(full_bar + 8 * stage, phase, abort_flag, F_WAIT_BUDGET)) {
          *abort_flag = 1;
          atomicCAS(p.status, 0, MB_DEV_TIMEOUT_EPILOGUE);
          ok = false;
          break;
        }
        if (warp == 2 && lane == 0) MBF_STAMP_K(1, kstep);
        // The slot's previous contents are dead: the producer refilled this stage only after
        // the MMAs that read the slot had completed.
        tc_fence_after_sync();
        const float *xs = reinterpret_cast<const float *>(smem_aligned + stage * Cfg::STAGE_BYTES) +
                          quarter * 32 + lane;
        const uint32_t a_col = tmem_base + a_lane + Cfg::A_COL0 + stage * F_A_COLS;
#pragma unroll
        for (int h = 0; h < FKB / 16; ++h) {
          uint32_t hi[16], lo[16];
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const uint32_t v = __float_as_uint(xs[(h * 16 + k) * FBM]);
            hi[k] = v & 0xffffe000u;
            lo[k] = __float_as_uint(__uint_as_float(v) - __uint_as_float(hi[k]));
          }
          tmem_st_32x32b_x16(a_col + h * 16, hi);
          tmem_st_32x32b_x16(a_col + FKB + h * 16, lo);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(split_bar + 8 * stage);
        if (warp == 2 && lane == 0) MBF_STAMP_K(2, kstep);
        ++kstep;
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp < F_FIRST_EPI_WARP) {
    // ---------------- W split: hi / lo tiles in shared memory ----------------
    const int t = (warp - F_FIRST_WSPLIT_WARP) * 32 + lane;  // 0..127
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int kstep = 0;
    for (FTileIter it(p); ok && it.valid(p); it.next(p)) {
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait_warp(full_bar + 8 * stage, phase, abort_flag, F_WAIT_BUDGET)) {
          *abort_flag = 1;
          atomicCAS(p.status, 0, MB_DEV_TIMEOUT_EPILOGUE);
          ok = false;
          break;
        }
        uint4 *hi = reinterpret_cast<uint4 *>(smem_aligned + stage * Cfg::STAGE_BYTES + Cfg::X_BYTES);
        uint4 *lo = hi + Cfg::W_BYTES / 16;
        // the split is element-wise, so the swizzled placement does not matter
#pragma unroll
        for (int i = 0; i < Cfg::W_BYTES / 16 / (F_WSPLIT_WARPS * 32); ++i) {
          const uint4 v = hi[t + i * (F_WSPLIT_WARPS * 32)];
          uint4 h, l;
          h.x = v.x & 0xffffe000u; h.y = v.y & 0xffffe000u;
          h.z = v.z & 0xffffe000u; h.w = v.w & 0xffffe000u;
          l.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(h.x));
          l.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(h.y));
          l.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(h.z));
          l.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(h.w));
          hi[t + i * (F_WSPLIT_WARPS * 32)] = h;
          lo[t + i * (F_WSPLIT_WARPS * 32)] = l;
        }
        fence_proxy_async();  // the MMA reads these tiles through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(split_bar + 8 * stage);
        if (t == 0) MBF_STAMP_K(5, kstep);
        ++kstep;
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
    const int my_turn = (warp - F_FIRST_EPI_WARP) & 3;  // which of the set's stores this warp issues
    constexpr int CHUNKS = BN / 16 / 2;              // 16-column chunks per warp
    // The activation as clamp + negative-slope term, with the choice made once: a branch
    // per value costs more than the arithmetic (few warps are there to hide its latency).
    //   NOOP: [-inf, inf], 0   RELU: [0, inf], 0   RELUX: [0, max_limit], 0   LEAKYRELU: [0, inf], coef
    const float act_lo = p.act == 0 ? -INFINITY : 0.f;
    const float act_hi = p.act == 2 ? p.max_limit : INFINITY;
    const float act_slope = p.act == 6 ? p.coef : 0.f;
    const bool leaky = p.act == 6;
    const float *__restrict__ bias = p.bias;
    const bool has_bias = bias != nullptr;
    const float *__restrict__ residual = p.residual;
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
      // Bias: lane j of a warp fetches the value of the chunk's channel j one chunk ahead and
      // the chunk broadcasts it with shuffles.  (A load per value needs a bounds branch per
      // value, and with eight warps nothing hides a branch: that form took 750 cycles a chunk.)
      float b_next = 0.f;
      if (has_bias) b_next = bias[min(n_first + (lane & 15), Ndim - 1)];
      // Residual (a tensor laid out like C, e.g. a bottleneck block's shortcut): the 16 values
      // of a chunk are requested one chunk ahead, from addresses clamped into the tensor
      // instead of guarded by branches; a lane's loads of one channel are 128 contiguous bytes
      // across the warp.
      const float *res = residual != nullptr
                             ? residual + it.b * p.c_batch_stride + min(m, p.Mdim - 1)
                             : nullptr;
      float r_next[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) r_next[j] = 0.f;
      if (res != nullptr) {
        // ask L2 for the NEXT tile's residual rows now (lane j: the 128-byte piece of channel j
        // of each chunk), a whole tile ahead of the loads that will want them
        FTileIter nit = it;
        nit.next(p);
        if (nit.valid(p) && lane < 16) {
          const float *nres = residual + nit.b * p.c_batch_stride +
                              min(static_cast<int64_t>(nit.tm) * FBM + quarter * 32, p.Mdim - 1);
          const int64_t nn = static_cast<int64_t>(nit.tn) * BN + set * (BN / 2) + lane;
#pragma unroll
          for (int c = 0; c < CHUNKS; ++c)
            prefetch_l2(nres + min(nn + c * 16, Ndim - 1) * p.c_row_stride);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) r_next[j] = __ldg(res + min(n_first + j, Ndim - 1) * p.c_row_stride);
      }
      // staging, per set of four warps: [buffer][channel j][128 pixels]; a lane's 16 writes of
      // a chunk go to 16 different rows, a warp's write of one row covers all 32 banks.  The
      // four warps fill one [16 x 128] tile together and one thread stores it with a single
      // TMA store of 512-byte rows (stores of 128-byte rows, one per warp, ran at half the rate).
      float *stage_f = reinterpret_cast<float *>(smem_aligned + STAGES * Cfg::STAGE_BYTES) +
                       set * (2 * 16 * FBM);
      const int m0 = it.tm * FBM;
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
        const float b_cur = b_next;
        if (has_bias && i + 1 < CHUNKS) b_next = bias[min(n0 + 16 + (lane & 15), Ndim - 1)];
        float r_cur[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) r_cur[j] = r_next[j];
        if (res != nullptr && i + 1 < CHUNKS) {
#pragma unroll
          for (int j = 0; j < 16; ++j) r_next[j] = __ldg(res + min(n0 + 16 + j, Ndim - 1) * p.c_row_stride);
        }
        float v[16];
        if constexpr (EPI == 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[i & 1][j]);
        } else if constexpr (EPI == 2) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float bj = __shfl_sync(0xffffffffu, b_cur, j);
            const float x = (__uint_as_float(r[i & 1][j]) + bj) + r_cur[j];
            v[j] = fminf(fmaxf(x, act_lo), act_hi);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float bj = __shfl_sync(0xffffffffu, b_cur, j);
            // (acc + bias) + residual: the rounding order of a convolution followed by a sum
            const float x = (__uint_as_float(r[i & 1][j]) + bj) + r_cur[j];
            const float neg = leaky ? fminf(x, 0.f) * act_slope : 0.f;
            v[j] = fminf(fmaxf(x, act_lo), act_hi) + neg;
          }
        }
        if (c_tma) {
          float *buf = stage_f + (i & 1) * (16 * FBM);
#pragma unroll
          for (int j = 0; j < 16; ++j) buf[j * FBM + quarter * 32 + lane] = v[j];
          fence_proxy_async();
          // The four warps of a set take turns at issuing the stores (an issue costs its thread
          // some 200 cycles; on one fixed thread that would be on every chunk's critical path).
          // Before the barrier the thread that issued the previous store makes sure that it has
          // read its buffer: after the barrier this buffer is complete AND the other one is free.
          const int turn = (local * CHUNKS + i) & 3;
          if (lane == 0 && my_turn == ((turn + 3) & 3)) bulk_wait_group_read<0>();
          named_bar_sync(1 + set, 128);
          if (lane == 0 && my_turn == turn && n0 < p.Ndim) {
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

template <int BN, int EPI = 0>
int launch_f32(mb_context *ctx, const CUtensorMap &tx, const CUtensorMap &tw, const CUtensorMap &tc,
               F32TcParams &p, int cfg_bit) {
  using Cfg = F32Cfg<BN>;
  auto kern = gemm_f32_tc_kernel<BN, EPI>;
  uint64_t &mask = EPI != 0 ? ctx->func_attr_mask2 : ctx->func_attr_mask;
  if (!(mask & (1ull << (cfg_bit + 2 * EPI)))) {
    MB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    mask |= (1ull << (cfg_bit + 2 * EPI));
  }
  const int64_t total = p.batch * p.tiles_m * p.tiles_n;
  const int grid = static_cast<int>(total < ctx->num_sms ? total : ctx->num_sms);
  p.step_m = grid % p.tiles_m;
  p.step_n = (grid / p.tiles_m) % p.tiles_n;
  p.step_b = (grid / p.tiles_m) / p.tiles_n;
  MB_CUDA(ctx, mb_launch_chained(ctx, kern, dim3(grid), dim3(F_THREADS), Cfg::SMEM_BYTES, tx, tw, tc, p));
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
                          float coef, const float *residual) {
  const int BN = Ndim > 64 ? 128 : 64;
  F32TcParams p;
  p.Mdim = Mdim; p.Ndim = Ndim; p.K = K; p.batch = batch;
  p.tiles_m = static_cast<int>(ceil_div64(Mdim, FBM));
  p.tiles_n = static_cast<int>(ceil_div64(Ndim, BN));
  p.k_blocks = static_cast<int>(ceil_div64(K, FKB));
  p.x_batched = x_batch_stride != 0; p.w_batched = w_batch_stride != 0;
  p.bias = bias; p.residual = residual; p.act = act; p.max_limit = max_limit; p.coef = coef;
  p.C = C; p.c_row_stride = c_row_stride; p.c_batch_stride = c_batch_stride;
  p.status = ctx->dev_status;
  p.timeline = ctx->tc_timeline;
  CUtensorMap tx, tw;
  MB_RETURN_IF_ERROR(make_map_f32(ctx, &tx, X, Mdim, K, p.x_batched ? batch : 1, x_row_stride,
                                  p.x_batched ? x_batch_stride : x_row_stride * K, FBM, FKB,
                                  CU_TENSOR_MAP_SWIZZLE_NONE));
  MB_RETURN_IF_ERROR(make_map_f32(ctx, &tw, W, K, Ndim, p.w_batched ? batch : 1, w_row_stride,
                                  p.w_batched ? w_batch_stride : w_row_stride * Ndim, FKB, BN));
  CUtensorMap tc;
  p.c_tma = ((reinterpret_cast<uintptr_t>(C) & 15u) == 0 && c_row_stride % 4 == 0 &&
             c_batch_stride % 4 == 0 && Ndim >= 16) ? 1 : 0;
  if (p.c_tma) {
    MB_RETURN_IF_ERROR(make_map_f32(ctx, &tc, C, Mdim, Ndim, batch, c_row_stride,
                                    batch > 1 ? c_batch_stride : c_row_stride * Ndim, FBM, 16,
                                    CU_TENSOR_MAP_SWIZZLE_NONE));
  } else {
    memset(&tc, 0, sizeof(tc));
  }
  if (bias == nullptr && residual == nullptr && act == 0) {
    if (BN == 128) return launch_f32<128, 1>(ctx, tx, tw, tc, p, 41);
    return launch_f32<64, 1>(ctx, tx, tw, tc, p, 42);
  }
  if (act != 6) {
    if (BN == 128) return launch_f32<128, 2>(ctx, tx, tw, tc, p, 41);
    return launch_f32<64, 2>(ctx, tx, tw, tc, p, 42);
  }
  if (BN == 128) return launch_f32<128>(ctx, tx, tw, tc, p, 41);
  return launch_f32<64>(ctx, tx, tw, tc, p, 42);
}
