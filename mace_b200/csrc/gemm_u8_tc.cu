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
// Structure (one persistent CTA per SM, 704 threads):
//   warp 0       TMA producer: 128-byte-swizzled tiles of A and B into a
//                multi-stage shared-memory ring (mbarrier full/empty pairs)
//   warp 1       MMA issuer: one thread issues tcgen05.mma 128 x BN x 32 steps
//                into one of two TMEM accumulator buffers
//   warps 2..5   preparation: per tile, the row and column terms of the
//                epilogue (zero-point corrections, bias) into shared memory.
//                With FUSE_SUMS they also add up the operand bytes of every
//                stage straight from the tiles in shared memory, so the
//                correction needs no extra pass over the operands; that mode
//                serves K-major operands with K <= 1024 (pointwise
//                convolutions), where the tensor pipe has time to spare.
//                Large-K GEMMs take their sums from separate kernels, because
//                the extra shared-memory reads would slow their main loop.
//   warps 6..21  epilogue: sets of four warps (one per TMEM lane quarter), each set on
//                a 64-column slice of a tile; BN / 64 sets share a tile and the other
//                sets drain the following tiles from their own accumulator buffers.
//                Per 16-column chunk: tcgen05.ld (the next chunk is in flight while
//                the current one is processed), add the terms, requantize (one 64-bit
//                multiply-add per value), pack; two chunks are staged in shared memory
//                (32 rows x 32 bytes, 32-byte swizzle) and written by one TMA store,
//                which also clips the ragged edges of M and N.  Outputs TMA cannot
//                address (int32, unaligned rows) take plain stores.
//   K <= 64      K-major operands use 64- or 32-byte rows (64B / 32B swizzle) so that
//                the TMA boxes of the first pointwise convolutions carry no padding.
// Every wait is bounded; on a timeout the kernel records a status word, lets
// outstanding copies land, frees its TMEM and returns.
#include <algorithm>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128;        // rows of A per tile == TMEM lanes
constexpr int BK = 128;        // bytes of K per pipeline stage (one swizzle row); K-major
                               // operands with K <= 64 use rows of 64 or 32 bytes (template KB)
constexpr int UMMA_K = 32;     // K per tcgen05.mma for 8-bit operands
constexpr int PREP_WARPS = 4;
constexpr int EPI_WARPS = 16;
constexpr int FIRST_EPI_WARP = 2 + PREP_WARPS;
constexpr int NUM_THREADS = (2 + PREP_WARPS + EPI_WARPS) * 32;
constexpr int CHUNK = 16;      // accumulator columns per tcgen05.ld
constexpr long long WAIT_BUDGET = 1ll << 31;  // ~1 s of SM clocks per wait
constexpr uint32_t SWIZZLE_128B = 2;

struct TcParams {
  int64_t M, N, K, batch;
  int tiles_m, tiles_n, k_blocks;
  int64_t total_tiles;

  // gridDim.x as (step_b, step_n, step_m) in tile coordinates: advancing a CTA to its next
  // tile is three additions and two carries instead of 64-bit divisions
  int step_m, step_n, step_b;
  // Operand byte sums, each as `slices` partial rows that are added up here:
  const uint32_t *sum_a;  // [batch or 1][sum_a_slices][M]; null when fused or zp_b == 0
  const uint32_t *sum_b;  // [batch or 1][sum_b_slices][N]; null when fused or zp_a == 0
  int64_t sum_a_bstride, sum_b_bstride;
  int sum_a_slices, sum_b_slices;
  int a_batched, b_batched;
  const int32_t *bias;
  int bias_per_row;
  int32_t zp_a, zp_b, kzz;
  mb_requant_params rq;
  int rq_variant;  // mb_requant_variant() (0..5), or 8 = the Gemv delegators' float rule
                   // (mult_f, zp_f)
  float mult_f, zp_f;
  void *C;
  int out_is_int32;
  int c_tma;  // uint8 C written by TMA stores (base and rows 16-byte aligned)
  // The kernel in front of this one in the stream only computes sum_a / sum_b (the operands
  // themselves were complete before it started): the main loop starts without waiting for it,
  // only the preparation warps wait, where they read the sums.
  int sums_pending;
  int b_const;  // B is a weight: its first tiles may be asked into L2 before the wait for the kernel in front
  int *status;
  // null, or clock stamps written by CTA 0 (profiling aid): 32 milestone slots, then 5
  // slots for each of its first 16 tiles (TMA issued, tile landed, MMAs committed,
  // epilogue begins, epilogue ends); the buffer holds 128 values
  long long *timeline;
};

// Clock stamp of a pipeline milestone, CTA 0 only, when a buffer was given.  Compiled in
// only with -DMB_TC_TIMELINE: the checks sit on the single-thread roles' critical path.
#ifdef MB_TC_TIMELINE
#define MB_STAMP(slot)                                                    \
  do {                                                                    \
    if (p.timeline != nullptr && blockIdx.x == 0) p.timeline[slot] = clock64(); \
  } while (0)
#else
#define MB_STAMP(slot) do { } while (0)
#endif

// Per-tile stamp k (0..4) of CTA 0's n-th tile, first 16 tiles only.
#ifndef MB_TC_TIMELINE
#define MB_STAMP_TILE(tile, k) do { (void)(tile); } while (0)
#else
#define MB_STAMP_TILE(tile, k)                                                       \
  do {                                                                              \
    if (p.timeline != nullptr && blockIdx.x == 0 && (tile) < 16)                    \
      p.timeline[32 + (tile) * 5 + (k)] = clock64();                                \
  } while (0)
#endif

// TCR ("row sums on the tensor core"): the B tile of every stage is followed by 16 constant rows
// of ones, and the MMA runs with N = BN + 16: accumulator columns BN .. BN + 15 of row m then
// hold the byte sum of A's row m, which the zero-point correction needs, at the price of an
// eighth (BN = 128) or a quarter (BN = 64) more work for a tensor pipe that short-K tiles leave
// idle anyway -- instead of a pass of the preparation warps over every A tile in shared memory,
// which cost these issue-bound kernels a fifth of their instructions.
// PAIR: two CTAs of a cluster work on one 256 x 256 tile: each holds 128 rows of A and 128 of
// the 256 columns of B in its shared memory (two thirds of the operand bytes per row of C that
// a lone CTA pulls for 128 x 256), and its own 128 rows of the accumulator in its tensor memory.
template <int BN, bool B_MN, int KB = BK, bool TCR = false, bool PAIR = false>
struct TileCfg {
  static_assert(!PAIR || (BN == 256 && KB == 128 && !TCR), "pairs: 256 columns, 128-byte rows");
  static_assert(KB == 128 || !B_MN, "short rows are for K-major operands");
  static_assert(!TCR || (!B_MN && BN <= 128), "ones rows follow a K-major B tile of at most 128 rows");
  static constexpr int BNX = TCR ? BN + 16 : BN;  // MMA N and TMEM columns per accumulator
  static constexpr int A_BYTES = BM * KB;
  static constexpr int B_TMA_BYTES = PAIR ? 128 * KB : B_MN ? ((BN + 127) / 128) * 128 * KB : BN * KB;  // what TMA brings
  static constexpr int B_BYTES = B_TMA_BYTES + (TCR ? 16 * KB : 0);
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGE_TX = A_BYTES + B_TMA_BYTES;
  // epilogue staging for the TMA stores: 1 KB (32 rows x 32 bytes) per epilogue warp
  // ... 2 KB (32 rows x 64 bytes: one store per warp and tile) where the ring leaves room
  static constexpr int STG_CHUNKS = BN == 256 ? 2 : 4;   // 16-byte chunks per staged row
  static constexpr int STAGING_BYTES = EPI_WARPS * 32 * STG_CHUNKS * 16;
  static constexpr int RING_BUDGET = 208 * 1024 - STAGING_BYTES;
  static constexpr int STAGES = RING_BUDGET / STAGE_BYTES > 8 ? 8 : RING_BUDGET / STAGE_BYTES;
  // all 512 TMEM columns as accumulator buffers: 2 for BN = 256, 4 for 128, 8 for 64, so
  // that narrow tiles (short main loops) keep several tiles in flight
  static constexpr int NUM_ACC = 512 / BNX;
  static constexpr int TMEM_COLS = 512;
  static constexpr int BAR_BYTES = 512;
  // + for a row-major B: the preparation warps' partial column sums, [tile parity][k quarter][columns]
  static constexpr int PART_INTS = B_MN ? 4 * ((BN + 127) / 128) * 128 : 0;
  static constexpr int TERM_BYTES = NUM_ACC * (128 + BN) * 4 + 2 * PART_INTS * 4;
  static constexpr int SMEM_BYTES =
      STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /*align*/ + BAR_BYTES + TERM_BYTES;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

// Adds up the `slices` partial rows of an operand sum for one row / column: eight loads in
// flight at a time (one after the other they would cost an L2 round trip each, and the terms
// of a tile have to be ready within the tile's main loop).
__device__ __forceinline__ uint32_t sum_partials(const uint32_t *p, int slices, int64_t stride) {
  uint32_t a0 = 0, a1 = 0, a2 = 0, a3 = 0, a4 = 0, a5 = 0, a6 = 0, a7 = 0;
  int sl = 0;
  for (; sl + 8 <= slices; sl += 8) {
    const uint32_t *q = p + sl * stride;
    const uint32_t v0 = __ldg(q), v1 = __ldg(q + stride), v2 = __ldg(q + 2 * stride), v3 = __ldg(q + 3 * stride);
    const uint32_t v4 = __ldg(q + 4 * stride), v5 = __ldg(q + 5 * stride), v6 = __ldg(q + 6 * stride),
                   v7 = __ldg(q + 7 * stride);
    a0 += v0; a1 += v1; a2 += v2; a3 += v3; a4 += v4; a5 += v5; a6 += v6; a7 += v7;
  }
  for (; sl < slices; ++sl) a0 += __ldg(p + sl * stride);
  return ((a0 + a1) + (a2 + a3)) + ((a4 + a5) + (a6 + a7));
}

__device__ __forceinline__ uint32_t sum16(const uint4 v, uint32_t s) {
  s = __dp4a(v.x, 0x01010101u, s);
  s = __dp4a(v.y, 0x01010101u, s);
  s = __dp4a(v.z, 0x01010101u, s);
  return __dp4a(v.w, 0x01010101u, s);
}

// Tile coordinates of a persistent CTA: tile index = (b * tiles_n + tn) * tiles_m + tm,
// advanced by gridDim.x per step.
struct TileIter {
  int tm, tn, b;
  __device__ __forceinline__ TileIter(const TcParams &p, bool pair = false) {
    const unsigned t = pair ? blockIdx.x >> 1 : blockIdx.x;  // < tiles of the first wave, one division pair per kernel
    tm = t % p.tiles_m;
    const unsigned q = t / p.tiles_m;
    tn = q % p.tiles_n;
    b = q / p.tiles_n;
  }
  __device__ __forceinline__ bool valid(const TcParams &p) const { return b < p.batch; }
  __device__ __forceinline__ void next(const TcParams &p) {
    tm += p.step_m;
    tn += p.step_n;
    b += p.step_b;
    if (tm >= p.tiles_m) { tm -= p.tiles_m; ++tn; }
    if (tn >= p.tiles_n) { tn -= p.tiles_n; ++b; }
  }
};

// Requantizes one 16-column chunk of an accumulator row and packs it into four words.
// MODE: 0..3 = mb_requant_t<ZP0 = bit 0, SGE1 = bit 1>; 4 / 5 = packed saturating form
// (zero point != 0 / == 0); 8 = the Gemv delegators' float rule.
template <int MODE>
__device__ __forceinline__ void requant_chunk(const uint32_t (&raw)[CHUNK], int32_t row_term,
                                              const int4 *ct, const TcParams &p,
                                              uint32_t (&packed)[CHUNK / 4]);

// The float rule of the Gemv delegators (mace/ops/arm/q8/gemv.cc:151-164):
// Saturate<uint8_t>(roundf(acc * multiplier [+ zp_out])), product and sum rounded separately
// (zp_f is 0 for the REF delegator's formula, which omits the zero point).
__device__ __forceinline__ uint32_t requant_float_rule(int32_t acc, float mult_f, float zp_f) {
  const float v = __fadd_rn(__fmul_rn(static_cast<float>(acc), mult_f), zp_f);
  return mb_saturate_round_u8(v);
}

template <int MODE>
__device__ __forceinline__ void requant_chunk(const uint32_t (&raw)[CHUNK], int32_t row_term,
                                              const int4 *ct, const TcParams &p,
                                              uint32_t (&packed)[CHUNK / 4]) {
#pragma unroll
  for (int q = 0; q < CHUNK / 4; ++q) {
    const int4 t = ct[q];  // broadcast read: all lanes, same address
    const int32_t a0 = static_cast<int32_t>(raw[4 * q + 0]) + row_term + t.x;
    const int32_t a1 = static_cast<int32_t>(raw[4 * q + 1]) + row_term + t.y;
    const int32_t a2 = static_cast<int32_t>(raw[4 * q + 2]) + row_term + t.z;
    const int32_t a3 = static_cast<int32_t>(raw[4 * q + 3]) + row_term + t.w;
    if (MODE == 4 || MODE == 5) {
      packed[q] = mb_requant_pack4<MODE == 5>(a0, a1, a2, a3, p.rq);
    } else {
      uint32_t b0, b1, b2, b3;
      if (MODE == 8) {
        b0 = requant_float_rule(a0, p.mult_f, p.zp_f); b1 = requant_float_rule(a1, p.mult_f, p.zp_f);
        b2 = requant_float_rule(a2, p.mult_f, p.zp_f); b3 = requant_float_rule(a3, p.mult_f, p.zp_f);
      } else {
        b0 = mb_requant_t<(MODE & 1) != 0, (MODE & 2) != 0>(a0, p.rq);
        b1 = mb_requant_t<(MODE & 1) != 0, (MODE & 2) != 0>(a1, p.rq);
        b2 = mb_requant_t<(MODE & 1) != 0, (MODE & 2) != 0>(a2, p.rq);
        b3 = mb_requant_t<(MODE & 1) != 0, (MODE & 2) != 0>(a3, p.rq);
      }
      packed[q] = __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
    }
  }
}

// What an epilogue warp needs for one tile on the TMA-store path.
struct EpiTile {
  uint32_t tbase;          // TMEM address of the warp's 32 lanes x 64 columns
  int32_t row_term;
  const int32_t *ct_base;  // column terms of the 64 columns (shared memory)
  uint32_t tempty;         // barrier that returns the accumulator buffer
  uint32_t tempty_leader;  // pairs, odd CTA: the even CTA's barrier too (shared::cluster address)
  uint4 *stage_row;        // this lane's row of the staging buffer (STG chunks of 16 bytes)
  int swz;
  uint32_t stage_addr;
  int64_t n_first;
  int m0, b, lane;
};

// 32 rows x 64 columns of one tile: four 16-column chunks from TMEM (the next one in flight
// while the current one is requantized), staged STG chunks at a time for a TMA store of
// 32 rows x 16*STG bytes.
template <int STG, int MODE, bool PAIR = false>
__device__ __forceinline__ void epi_tma_tile(const EpiTile &e, const CUtensorMap &tmap_c,
                                             const TcParams &p) {
  uint32_t r[2][CHUNK];
  tmem_ld_32x32b_x16(e.tbase, r[0]);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    tmem_ld_wait_x16(r[i & 1]);
    if (i + 1 < 4) tmem_ld_32x32b_x16(e.tbase + (i + 1) * CHUNK, r[(i + 1) & 1]);
    uint32_t packed[CHUNK / 4];
    requant_chunk<MODE>(r[i & 1], e.row_term, reinterpret_cast<const int4 *>(e.ct_base + i * CHUNK), p, packed);
    if (i == 3) {
      // The accumulator is in registers and the tile's terms have been read: hand the buffer
      // (TMEM columns and term slots; the preparation warps refill the latter on the same
      // barrier) back before the staging and the store.
      tc_fence_before_sync();
      __syncwarp();
      if (e.lane == 0) {
        mbar_arrive(e.tempty);
        if (PAIR && e.tempty_leader != 0) mbar_arrive_cluster(e.tempty_leader);
      }
    }
    if ((i & (STG - 1)) == 0) {
      // the previous store must have read the staging buffer before it is refilled
      if (e.lane == 0) bulk_wait_group_read<0>();
      __syncwarp();
    }
    e.stage_row[(i & (STG - 1)) ^ e.swz] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    if ((i & (STG - 1)) == STG - 1) {
      fence_proxy_async();
      __syncwarp();
      const int64_t n0 = e.n_first + (i - (STG - 1)) * CHUNK;
      if (e.lane == 0 && n0 < p.N && e.m0 < p.M) {
        tma_store_3d(&tmap_c, e.stage_addr, static_cast<int>(n0), e.m0, e.b);
        bulk_commit_group();
      }
    }
  }
}

template <int BN, bool A_MN, bool B_MN, bool FUSE_SUMS, int KB, bool TCR_ON = false, bool PAIR = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_u8_tc_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_c, const TcParams p) {
  constexpr bool TCR = TCR_ON && FUSE_SUMS && BN <= 128;
  static_assert(!PAIR || !FUSE_SUMS, "pairs take their operand sums from the sums kernel");
  using Cfg = TileCfg<BN, B_MN, KB, TCR, PAIR>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int TILE_M = PAIR ? 2 * BM : BM;  // rows of C per tile (of the pair)
  // pairs: the even CTA issues the MMAs for both; rank is this CTA's half of the rows and columns
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  constexpr int BNX = Cfg::BNX;
  // the preparation warps read the operand tiles in shared memory only for the sums the tensor
  // core does not deliver: B's (needed when zp_a != 0), and A's without the ones rows
  const bool prep_reads_tiles = FUSE_SUMS && ((!TCR && p.zp_b != 0) || p.zp_a != 0);
  // shared-memory descriptor fields for rows of KB bytes: swizzle mode and the distance
  // between 8-row groups
  constexpr uint32_t SWZ = KB == 128 ? 2u : KB == 64 ? 4u : 6u;
  constexpr uint32_t SBO = 8 * KB;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  // barrier block after the tile ring
  uint64_t *bars =
      reinterpret_cast<uint64_t *>(smem_aligned + STAGES * Cfg::STAGE_BYTES + Cfg::STAGING_BYTES);
  const uint32_t full_bar = smem_u32(bars);                  // [STAGES] tile landed
  const uint32_t empty_bar = full_bar + 8 * STAGES;          // [STAGES] tile consumed
  constexpr int NUM_ACC = Cfg::NUM_ACC;
  const uint32_t tfull_bar = empty_bar + 8 * STAGES;         // [NUM_ACC] accumulator complete
  const uint32_t tempty_bar = tfull_bar + 8 * NUM_ACC;       // [NUM_ACC] accumulator drained
  const uint32_t terms_bar = tempty_bar + 8 * NUM_ACC;       // [NUM_ACC] epilogue terms ready
  const uint32_t part_bar = terms_bar + 8 * NUM_ACC;          // the four quarters of a tile's column sums are written
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 3 * NUM_ACC + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  // per accumulator buffer: row terms [128] and column terms [BN]
  int32_t *row_term_sm =
      reinterpret_cast<int32_t *>(smem_aligned + STAGES * Cfg::STAGE_BYTES + Cfg::STAGING_BYTES +
                                  Cfg::BAR_BYTES);
  int32_t *col_term_sm = row_term_sm + NUM_ACC * 128;
  uint32_t *part_sm = reinterpret_cast<uint32_t *>(col_term_sm + NUM_ACC * BN);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  mb_grid_dep_launch();  // the kernel behind this one may start its own prologue

  if (threadIdx.x == 0) {
    MB_STAMP(0);
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    if (p.c_tma) prefetch_tensormap(&tmap_c);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, prep_reads_tiles ? 1 + PREP_WARPS : 1);
    }
    mbar_init(part_bar, PREP_WARPS);
    for (int b = 0; b < NUM_ACC; ++b) {
      mbar_init(tfull_bar + 8 * b, 1);
      // (pairs: the even CTA's barrier also counts the odd CTA's epilogue warps)
      mbar_init(tempty_bar + 8 * b, (PAIR && rank == 0 ? 2 : 1) * 4 * (BN / 64));
      mbar_init(terms_bar + 8 * b, PREP_WARPS);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_slot), Cfg::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
      tmem_relinquish();
    }
  }
  if (TCR) {
    // the 16 rows of ones behind every stage's B tile (TMA never writes there)
    constexpr int ONES_VECS = 16 * KB / 16;
    for (int i = threadIdx.x; i < STAGES * ONES_VECS; i += NUM_THREADS) {
      const int st = i / ONES_VECS, v = i - st * ONES_VECS;
      *reinterpret_cast<uint4 *>(smem_aligned + st * Cfg::STAGE_BYTES + Cfg::A_BYTES + Cfg::B_TMA_BYTES + v * 16) =
          make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
    }
    fence_proxy_async();  // generic-proxy writes, read by the tensor core through the async proxy
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // both CTAs' barriers exist before either arrives on the other's
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) MB_STAMP(1);
  // Everything above touched only this CTA's shared and tensor memory (and the kernel's
  // parameters); from here on the roles read and write global memory, which the kernel in
  // front of this one in the stream may still be producing.
  // (with sums_pending only the preparation warps, which read the sums, wait; the operands were
  // complete before the sums kernel started, and C is not touched by it)
  if (!PAIR && p.b_const && warp == 0 && lane == 0) {
    // a weight matrix is usually not in L2 any more (the activations of a whole network pass have
    // gone through it since): ask for this CTA's first B tiles now, so that they travel from HBM
    // while the kernel in front finishes
    TileIter it(p, PAIR);
    if (it.valid(p)) {
      const int bb = p.b_batched ? it.b : 0;
      const int ahead = p.k_blocks < STAGES ? p.k_blocks : STAGES;
      for (int kb = 0; kb < ahead; ++kb) {
        if (B_MN) {
#pragma unroll
          for (int j = 0; j < (BN + 127) / 128; ++j) tma_prefetch_3d(&tmap_b, it.tn * BN + j * 128, kb * KB, bb);
        } else {
          tma_prefetch_3d(&tmap_b, kb * KB, it.tn * BN, bb);
        }
      }
    }
  }
  if (!p.sums_pending || (warp >= 2 && warp < 2 + PREP_WARPS)) mb_grid_dep_wait();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // One thread runs the role (see the MMA issuer); the other lanes wait at the warp barrier.
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;  // this CTA's tile counter (profiling stamps)
      // When every tile of the launch reads the same B tile (one column of tiles, one K step,
      // B shared by the batch: a pointwise convolution with few channels), each stage's copy
      // of B is loaded once, on the first pass through the ring, and then left in place: TMA
      // handles short rows one by one, and the B rows would be a third to a half of them.
      const bool b_once = p.tiles_n == 1 && p.k_blocks == 1 && !p.b_batched;
      for (TileIter it(p, PAIR); ok && it.valid(p); it.next(p), ++local) {
        const int b = it.b, tm = it.tm, tn = it.tn;
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
          const bool skip_b = b_once && local >= STAGES;
          if (PAIR) {
            // Both CTAs' bytes are counted on the even CTA's barrier, which its MMA thread
            // waits on: this CTA's 128 rows of A and 128 of the tile's 256 columns of B.
            if (rank == 0) mbar_arrive_expect_tx(fb, 2 * Cfg::STAGE_TX);
            const uint32_t fbc = mapa_shared(fb, 0);
            if (A_MN) tma_load_3d_pair(sa, &tmap_a, fbc, tm * TILE_M + rank * BM, kb * KB, ab);
            else tma_load_3d_pair(sa, &tmap_a, fbc, kb * KB, tm * TILE_M + rank * BM, ab);
            if (B_MN) tma_load_3d_pair(sb, &tmap_b, fbc, tn * BN + rank * 128, kb * KB, bb);
            else tma_load_3d_pair(sb, &tmap_b, fbc, kb * KB, tn * BN + rank * 128, bb);
          } else {
          mbar_arrive_expect_tx(fb, skip_b ? Cfg::A_BYTES : Cfg::STAGE_TX);
          if (A_MN) {
            tma_load_3d(sa, &tmap_a, fb, tm * BM, kb * KB, ab);
          } else {
            tma_load_3d(sa, &tmap_a, fb, kb * KB, tm * BM, ab);
          }
          if (skip_b) {
            // B of this stage is already in place
          } else if (B_MN) {
#pragma unroll
            for (int j = 0; j < (BN + 127) / 128; ++j)
              tma_load_3d(sb + j * 128 * KB, &tmap_b, fb, tn * BN + j * 128, kb * KB, bb);
          } else {
            tma_load_3d(sb, &tmap_b, fb, kb * KB, tn * BN, bb);
          }
          }
          if (local == 0) MB_STAMP(2 + (kb < 3 ? kb : 3));  // TMA of k-block kb issued
          if (kb == 0) MB_STAMP_TILE(local, 0);
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
    // One thread runs the whole role; the other lanes go straight to the warp barrier below.
    // What the thread does between two MMAs has to fit into the time the tensor pipe's short
    // queue keeps it busy, and for tiles of one K step it is on the critical path outright:
    // the descriptors are one add per step and nothing in the loop is warp-collective.
    if (PAIR && rank != 0) {
      // the odd CTA issues no MMAs: the even CTA's thread drives both tensor cores
    } else if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(/*c s32*/ 2, /*a u8*/ 0, /*b u8*/ 0, A_MN, B_MN, TILE_M, BNX);
      // K-major tile: rows of KB bytes, 8-row groups SBO bytes apart; a K step moves 32 bytes
      // inside the swizzled row.  MN-major tile: k-rows of 128 bytes (128 elements of M or N),
      // 8-k-row groups 1024 bytes apart, 128-element atoms 128 * KB bytes apart; a K step moves
      // 32 k-rows = 4096 bytes.  The address field counts 16-byte units.
      const uint64_t a_base = A_MN ? make_smem_desc(0, 128 * KB, 1024, SWIZZLE_128B) : make_smem_desc(0, 16, SBO, SWZ);
      const uint64_t b_base = B_MN ? make_smem_desc(0, 128 * KB, 1024, SWIZZLE_128B) : make_smem_desc(0, 16, SBO, SWZ);
      constexpr uint32_t a_step = (A_MN ? UMMA_K * 128 : UMMA_K) >> 4;
      constexpr uint32_t b_step = (B_MN ? UMMA_K * 128 : UMMA_K) >> 4;
      const int last_ksteps =
          static_cast<int>((p.K - static_cast<int64_t>(p.k_blocks - 1) * KB + UMMA_K - 1) / UMMA_K);
      int stage = 0;
      uint32_t phase = 0;
      int acc_buf = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      int local = 0;
      for (TileIter it(p, PAIR); ok && it.valid(p); it.next(p), ++local) {
        if (!mbar_wait(tempty_bar + 8 * acc_buf, acc_phase ^ 1, abort_flag, WAIT_BUDGET)) {
          *abort_flag = 1;
          atomicCAS(p.status, 0, MB_DEV_TIMEOUT_MMA);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc_buf * BNX;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, WAIT_BUDGET)) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, MB_DEV_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (local == 0) MB_STAMP(6 + (kb < 3 ? kb : 3));  // k-block kb landed
          if (kb == p.k_blocks - 1) MB_STAMP_TILE(local, 1);
          const uint32_t sa = smem_base + stage * Cfg::STAGE_BYTES;
          const uint64_t a_desc = a_base | static_cast<uint64_t>((sa >> 4) & 0x3FFFu);
          const uint64_t b_desc = b_base | static_cast<uint64_t>(((sa + Cfg::A_BYTES) >> 4) & 0x3FFFu);
          if (PAIR) {
            const int ksteps = (kb + 1 < p.k_blocks) ? KB / UMMA_K : last_ksteps;
            for (int j = 0; j < ksteps; ++j)
              mma_i8_ss_pair(d_tmem, a_desc + j * a_step, b_desc + j * b_step, idesc, (kb > 0 || j > 0) ? 1u : 0u);
            mma_commit_pair(empty_bar + 8 * stage, 3);  // frees the stage in both CTAs
          } else {
          if (kb + 1 < p.k_blocks || last_ksteps == KB / UMMA_K) {
#pragma unroll
            for (int j = 0; j < KB / UMMA_K; ++j)
              mma_i8_ss(d_tmem, a_desc + j * a_step, b_desc + j * b_step, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          } else {
            for (int j = 0; j < last_ksteps; ++j)
              mma_i8_ss(d_tmem, a_desc + j * a_step, b_desc + j * b_step, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          mma_commit(empty_bar + 8 * stage);  // frees the stage when the MMAs have read it
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (PAIR) mma_commit_pair(tfull_bar + 8 * acc_buf, 3);  // accumulator complete, in both CTAs
        else mma_commit(tfull_bar + 8 * acc_buf);               // accumulator complete
        if (local == 0) MB_STAMP(10);
        MB_STAMP_TILE(local, 2);
        if (++acc_buf == NUM_ACC) {
          acc_buf = 0;
          acc_phase ^= 1;
        }
      }
    }
    __syncwarp();
  } else if (warp < FIRST_EPI_WARP) {
    // ---------------- preparation: operand sums (fused) and epilogue terms ----------------
    const int r = (warp - 2) * 32 + lane;  // 0..127: row of the A tile / column slot
    int stage = 0;
    uint32_t phase = 0;
    int acc_buf = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    int local = 0;
    for (TileIter it(p, PAIR); ok && it.valid(p); it.next(p), ++local) {
      const int b = it.b, tm = it.tm, tn = it.tn;
      uint32_t sa_sum = 0, sb_sum[(BN + 127) / 128];
      uint32_t cs[(BN + 127) / 128][4];  // row-major B: four columns of each panel over this warp's k rows
#pragma unroll
      for (int j = 0; j < (BN + 127) / 128; ++j) {
        sb_sum[j] = 0;
        cs[j][0] = cs[j][1] = cs[j][2] = cs[j][3] = 0;
      }
      // global inputs of the terms, requested before the main loop is followed
      const int64_t m = static_cast<int64_t>(tm) * TILE_M + rank * BM + r;
      int32_t row_bias = 0, col_bias[(BN + 127) / 128];
      if (p.bias != nullptr && p.bias_per_row && m < p.M) row_bias = __ldg(p.bias + m);
      if (!FUSE_SUMS && p.sum_a != nullptr && m < p.M) {
        sa_sum = sum_partials(p.sum_a + (p.a_batched ? b : 0) * p.sum_a_bstride + m, p.sum_a_slices, p.M);
      }
#pragma unroll
      for (int j = 0; j < (BN + 127) / 128; ++j) {
        const int64_t n = static_cast<int64_t>(tn) * BN + j * 128 + r;
        col_bias[j] = (p.bias != nullptr && !p.bias_per_row && n < p.N) ? __ldg(p.bias + n) : 0;
        if (!FUSE_SUMS && p.sum_b != nullptr && n < p.N) {
          sb_sum[j] = sum_partials(p.sum_b + (p.b_batched ? b : 0) * p.sum_b_bstride + n, p.sum_b_slices, p.N);
        }
      }
      if (prep_reads_tiles) {
        const bool want_a = !TCR && p.zp_b != 0, want_b = p.zp_a != 0;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_warp(full_bar + 8 * stage, phase, abort_flag, WAIT_BUDGET)) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, MB_DEV_TIMEOUT_EPILOGUE);
            ok = false;
            break;
          }
          const uint8_t *ta = smem_aligned + stage * Cfg::STAGE_BYTES;
          const uint8_t *tb = ta + Cfg::A_BYTES;
          // a row is KB bytes = KB / 16 chunks of 16; start at chunk (r mod chunks) so that
          // the threads of a quarter warp spread over the bank groups.  The swizzle only
          // permutes chunks inside a row, which a sum does not see.
          if (want_a) {
#pragma unroll
            for (int i = 0; i < KB / 16; ++i)
              sa_sum = sum16(*reinterpret_cast<const uint4 *>(ta + r * KB + ((i + r) & (KB / 16 - 1)) * 16), sa_sum);
          }
#pragma unroll
          for (int j = 0; j < (BN + 127) / 128; ++j) {
            const int row = j * 128 + r;
            if (B_MN) {
              // The tile is [128-column panel][KB depth rows][128 bytes], the 16-byte chunks of a
              // row permuted by the row's low three bits.  Warp q takes depth rows 32 q .. 32 q + 31,
              // lane w the 32-bit word w of every such row (columns 4 w .. 4 w + 3 of the panel:
              // a warp reads a whole row per load, no conflicts), and adds the four bytes as two
              // pairs of 16-bit counts (32 rows x 255 fit); the four warps' counts meet below.
              if (want_b) {
                const int c = lane >> 2, q = warp - 2;
                const uint8_t *pan = tb + j * 128 * KB + q * 32 * 128 + (lane & 3) * 4;
                uint32_t ev = 0, od = 0;
                // (fully unrolled: the eight chunk offsets (c ^ 0..7) << 4 are computed once, every
                // load is register + immediate, two rows share one three-input add per count pair)
#pragma unroll
                for (int kk = 0; kk < 32; kk += 2) {
                  const uint32_t w0 = *reinterpret_cast<const uint32_t *>(pan + kk * 128 + ((c ^ (kk & 7)) << 4));
                  const uint32_t w1 =
                      *reinterpret_cast<const uint32_t *>(pan + (kk + 1) * 128 + ((c ^ ((kk + 1) & 7)) << 4));
                  ev += (w0 & 0x00ff00ffu) + (w1 & 0x00ff00ffu);
                  od += __byte_perm(w0, 0, 0x4341) + __byte_perm(w1, 0, 0x4341);
                }
                cs[j][0] += ev & 0xffffu;
                cs[j][1] += od & 0xffffu;
                cs[j][2] += ev >> 16;
                cs[j][3] += od >> 16;
              }
            } else if (want_b && row < BN) {
#pragma unroll
              for (int i = 0; i < KB / 16; ++i)
                sb_sum[j] = sum16(*reinterpret_cast<const uint4 *>(tb + row * KB + ((i + r) & (KB / 16 - 1)) * 16),
                                  sb_sum[j]);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(empty_bar + 8 * stage);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (B_MN && want_b) {
          // the four k quarters of every column: through shared memory (two buffers, by tile parity)
          constexpr int COLS = ((BN + 127) / 128) * 128;
          uint32_t *part = part_sm + (local & 1) * Cfg::PART_INTS;
#pragma unroll
          for (int j = 0; j < (BN + 127) / 128; ++j)
            *reinterpret_cast<uint4 *>(part + (warp - 2) * COLS + j * 128 + 4 * lane) =
                make_uint4(cs[j][0], cs[j][1], cs[j][2], cs[j][3]);
          __syncwarp();
          if (lane == 0) mbar_arrive(part_bar);
          if (!mbar_wait_warp(part_bar, static_cast<uint32_t>(local & 1), abort_flag, WAIT_BUDGET)) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, MB_DEV_TIMEOUT_EPILOGUE);
            break;
          }
#pragma unroll
          for (int j = 0; j < (BN + 127) / 128; ++j)
            sb_sum[j] = part[j * 128 + r] + part[COLS + j * 128 + r] + part[2 * COLS + j * 128 + r] +
                        part[3 * COLS + j * 128 + r];
        }
      }
      // terms of this tile (operand sums are zero where no correction is needed)
      const int32_t row_term = row_bias - p.zp_b * static_cast<int32_t>(sa_sum);
      int32_t col_term[(BN + 127) / 128];
#pragma unroll
      for (int j = 0; j < (BN + 127) / 128; ++j)
        col_term[j] = p.kzz + col_bias[j] - p.zp_a * static_cast<int32_t>(sb_sum[j]);
      // the terms of this buffer's previous tile must have been consumed
      if (!mbar_wait_warp(tempty_bar + 8 * acc_buf, acc_phase ^ 1, abort_flag, WAIT_BUDGET)) {
        *abort_flag = 1;
        atomicCAS(p.status, 0, MB_DEV_TIMEOUT_EPILOGUE);
        break;
      }
      row_term_sm[acc_buf * 128 + r] = row_term;
#pragma unroll
      for (int j = 0; j < (BN + 127) / 128; ++j)
        if (j * 128 + r < BN) col_term_sm[acc_buf * BN + j * 128 + r] = col_term[j];
      __syncwarp();
      if (lane == 0) mbar_arrive(terms_bar + 8 * acc_buf);
      if (local == 0 && warp == 2 && lane == 0) MB_STAMP(11);
      if (++acc_buf == NUM_ACC) {
        acc_buf = 0;
        acc_phase ^= 1;
      }
    }
  } else {
    // ---------------- epilogue ----------------
    // Four consecutive warps cover the four TMEM lane quarters of a 64-column slice of a
    // tile; BN / 64 such sets work on one tile, and the remaining sets on the tiles after
    // it (GROUPS tiles are drained at the same time, each from its own accumulator
    // buffer).  Per tile a warp handles 32 rows x 64 columns in four 16-column chunks.
    constexpr int SETS_PER_TILE = BN / 64;             // 1, 2, 4
    constexpr int GROUPS = 4 / SETS_PER_TILE;          // 4, 2, 1 tiles in flight
    constexpr int CHUNKS_PER_WARP = 4;
    const int quarter = warp & 3;                      // TMEM lanes [32*quarter, +32) are this warp's
    const int set = (warp - FIRST_EPI_WARP) >> 2;      // 0..3
    const int slice = set % SETS_PER_TILE;             // which 64 columns of the tile
    const int group = set / SETS_PER_TILE;             // which tiles: local % GROUPS == group
    // staging for the TMA store: 32 rows x 32 bytes (two chunks), 32-byte swizzle:
    // 16-byte half h of row r sits at r*32 + ((h ^ (r >> 2)) & 1)*16, which keeps the
    // quarter-warps' 16-byte writes free of bank conflicts
    constexpr int STG = Cfg::STG_CHUNKS;
    uint8_t *stage_ptr = smem_aligned + STAGES * Cfg::STAGE_BYTES + (warp - FIRST_EPI_WARP) * (32 * STG * 16);
    const uint32_t stage_addr = smem_u32(stage_ptr);
    uint4 *stage_row = reinterpret_cast<uint4 *>(stage_ptr + lane * (STG * 16));
    // 32-byte rows, 32-byte swizzle: half h of row r at ((h ^ (r >> 2)) & 1); 64-byte rows,
    // 64-byte swizzle: chunk c of row r at (c ^ (r >> 1)) & 3
    const int swz = STG == 2 ? ((lane >> 2) & 1) : ((lane >> 1) & 3);
    int local = 0;
    for (TileIter it(p, PAIR); it.valid(p); it.next(p), ++local) {
      if (local % GROUPS != group) continue;
      const int b = it.b, tm = it.tm, tn = it.tn;
      const int acc_buf = local % NUM_ACC;
      const uint32_t acc_phase = (local / NUM_ACC) & 1;
      if (!mbar_wait_warp(tfull_bar + 8 * acc_buf, acc_phase, abort_flag, WAIT_BUDGET) ||
          !mbar_wait_warp(terms_bar + 8 * acc_buf, acc_phase, abort_flag, WAIT_BUDGET)) {
        *abort_flag = 1;
        atomicCAS(p.status, 0, MB_DEV_TIMEOUT_EPILOGUE);
        break;
      }
      tc_fence_after_sync();
      if (local == 0 && warp == FIRST_EPI_WARP && lane == 0) MB_STAMP(12);
      if (warp == FIRST_EPI_WARP && lane == 0) MB_STAMP_TILE(local, 3);
      const int m0 = tm * TILE_M + rank * BM + quarter * 32;  // first row of this warp
      const int64_t m = static_cast<int64_t>(m0) + lane;
      const bool row_ok = m < p.M;
      int32_t row_term = row_term_sm[acc_buf * 128 + quarter * 32 + lane];
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc_buf * BNX +
                             slice * 64;
      if (TCR) {
        // columns BN .. BN + 15 of this lane's row: the byte sum of A's row (all 16 alike)
        uint32_t ones_cols[CHUNK];
        tmem_ld_32x32b_x16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc_buf * BNX + BN, ones_cols);
        tmem_ld_wait_x16(ones_cols);
        row_term -= p.zp_b * static_cast<int32_t>(ones_cols[0]);
      }
      const int32_t *ct_base = col_term_sm + acc_buf * BN + slice * 64;
      const int64_t n_first = static_cast<int64_t>(tn) * BN + slice * 64;
      if (p.c_tma) {
        // one decision per tile (not per chunk or value: with so few warps per scheduler
        // a branch's latency is not hidden)
        const EpiTile e{tbase, row_term, ct_base, tempty_bar + 8 * acc_buf,
                        (PAIR && rank != 0) ? mapa_shared(tempty_bar + 8 * acc_buf, 0) : 0u, stage_row, swz,
                        stage_addr, n_first, m0, b, lane};
        switch (p.rq_variant) {
          case 8: epi_tma_tile<STG, 8, PAIR>(e, tmap_c, p); break;
          case 5: epi_tma_tile<STG, 5, PAIR>(e, tmap_c, p); break;
          case 4: epi_tma_tile<STG, 4, PAIR>(e, tmap_c, p); break;
          case 3: epi_tma_tile<STG, 3, PAIR>(e, tmap_c, p); break;
          case 2: epi_tma_tile<STG, 2, PAIR>(e, tmap_c, p); break;
          case 1: epi_tma_tile<STG, 1, PAIR>(e, tmap_c, p); break;
          default: epi_tma_tile<STG, 0, PAIR>(e, tmap_c, p); break;
        }
      } else {
        // direct stores: int32 output, or a uint8 output whose rows TMA cannot address
        uint8_t *c8 = static_cast<uint8_t *>(p.C) + (static_cast<int64_t>(b) * p.M + m) * p.N;
        const bool words_ok = !p.out_is_int32 && (p.N & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 3u) == 0;
        int32_t *c32 = static_cast<int32_t *>(p.C) + (static_cast<int64_t>(b) * p.M + m) * p.N;
        const bool quads_ok = p.out_is_int32 && (p.N & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15u) == 0;
        uint32_t r[1][CHUNK];
        tmem_ld_32x32b_x16(tbase, r[0]);
#pragma unroll 1
        for (int i = 0; i < CHUNKS_PER_WARP; ++i) {
          uint32_t v[CHUNK];
          tmem_ld_wait_x16(r[0]);
#pragma unroll
          for (int j = 0; j < CHUNK; ++j) v[j] = r[0][j];
          if (i + 1 < CHUNKS_PER_WARP) tmem_ld_32x32b_x16(tbase + (i + 1) * CHUNK, r[0]);
          const int64_t n0 = n_first + i * CHUNK;
          const int32_t *ct = ct_base + i * CHUNK;
          if (words_ok && n0 + CHUNK <= p.N) {
            // a whole chunk of a uint8 row whose words are 4-byte aligned (N % 4 == 0, e.g. the
            // 1000 logits of a classifier, which TMA cannot address): requantize without a
            // branch per value and store four words instead of sixteen bytes
            uint32_t packed[CHUNK / 4];
            const int4 *ct4 = reinterpret_cast<const int4 *>(ct);
            switch (p.rq_variant) {
              case 8: requant_chunk<8>(v, row_term, ct4, p, packed); break;
              case 5: requant_chunk<5>(v, row_term, ct4, p, packed); break;
              case 4: requant_chunk<4>(v, row_term, ct4, p, packed); break;
              case 3: requant_chunk<3>(v, row_term, ct4, p, packed); break;
              case 2: requant_chunk<2>(v, row_term, ct4, p, packed); break;
              case 1: requant_chunk<1>(v, row_term, ct4, p, packed); break;
              default: requant_chunk<0>(v, row_term, ct4, p, packed); break;
            }
            if (row_ok) {
              uint32_t *cw = reinterpret_cast<uint32_t *>(c8 + n0);
#pragma unroll
              for (int q = 0; q < CHUNK / 4; ++q) cw[q] = packed[q];
            }
          } else if (quads_ok && n0 + CHUNK <= p.N) {
            // a whole chunk of an int32 row: four 16-byte stores instead of sixteen words
            if (row_ok) {
              int4 *cq = reinterpret_cast<int4 *>(c32 + n0);
#pragma unroll
              for (int q = 0; q < CHUNK / 4; ++q)
                cq[q] = make_int4(static_cast<int32_t>(v[4 * q + 0]) + row_term + ct[4 * q + 0],
                                  static_cast<int32_t>(v[4 * q + 1]) + row_term + ct[4 * q + 1],
                                  static_cast<int32_t>(v[4 * q + 2]) + row_term + ct[4 * q + 2],
                                  static_cast<int32_t>(v[4 * q + 3]) + row_term + ct[4 * q + 3]);
            }
          } else if (row_ok && n0 < p.N) {
#pragma unroll
            for (int j = 0; j < CHUNK; ++j) {
              const int32_t acc = static_cast<int32_t>(v[j]) + row_term + ct[j];
              if (n0 + j < p.N) {
                if (p.out_is_int32) c32[n0 + j] = acc;
                else c8[n0 + j] = static_cast<uint8_t>(p.rq_variant == 8 ? requant_float_rule(acc, p.mult_f, p.zp_f)
                                                                         : mb_requant_fast(acc, p.rq));
              }
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(tempty_bar + 8 * acc_buf);
          if (PAIR && rank != 0) mbar_arrive_cluster(mapa_shared(tempty_bar + 8 * acc_buf, 0));
        }
      }
      if (warp == FIRST_EPI_WARP && lane == 0) MB_STAMP(local == 0 ? 13 : 14);
      if (warp == FIRST_EPI_WARP && lane == 0) MB_STAMP_TILE(local, 4);
    }
    // the staging buffer must outlive the last store's read, and the kernel its writes
    if (lane == 0) bulk_wait_group<0>();
    __syncwarp();
  }

  __syncthreads();
  if (threadIdx.x == 0) MB_STAMP(15);
  if (*abort_flag != 0) {
    // Give copies and MMAs that are still in flight time to land before the
    // shared memory and TMEM they target go away (bounded: about 2 ms).
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  // pairs: neither CTA's shared or tensor memory may go away while the other can still reach
  // it (the even CTA's MMAs read the odd CTA's tiles; the odd CTA arrives on the even one's
  // barriers)
  if (PAIR) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 3-D uint8 tensor map: dims {inner, rows, batch}; 128-byte swizzle for the operand
// tiles, 32-byte swizzle for the output staging boxes.
int make_map_u8(mb_context *ctx, CUtensorMap *map, const void *base, uint64_t inner,
                uint64_t rows, uint64_t batch, uint64_t batch_stride_bytes, uint32_t box_inner,
                uint32_t box_rows, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B,
                uint64_t row_pitch = 0) {
  const cuuint64_t dims[3] = {inner, rows, batch};
  const cuuint64_t strides[2] = {row_pitch != 0 ? row_pitch : inner, batch_stride_bytes};
  const cuuint32_t box[3] = {box_inner, box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
      map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box, estr,
      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return mb_fail(ctx, MB_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
  return MB_SUCCESS;
}

template <int BN, bool A_MN, bool B_MN, bool FUSE_SUMS = false, int KB = BK, bool TCR_ON = false>
int launch_cfg(mb_context *ctx, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc,
               TcParams &p) {
  using Cfg = TileCfg<BN, B_MN, KB, TCR_ON && FUSE_SUMS && BN <= 128>;
  auto kern = gemm_u8_tc_kernel<BN, A_MN, B_MN, FUSE_SUMS, KB, TCR_ON>;
  // The opt-in shared-memory limit is a per-device function attribute; set it
  // once per context.
  constexpr int cfg_id = (BN == 256 ? 0 : BN == 128 ? 1 : 2) * 4 + (A_MN ? 2 : 0) + (B_MN ? 1 : 0) +
                         (FUSE_SUMS ? 12 : 0) + (KB == 64 ? 3 : KB == 32 ? 6 : 0) + (TCR_ON ? 24 : 0);
  if (!(ctx->func_attr_mask & (1ull << cfg_id))) {
    MB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      Cfg::SMEM_BYTES));
    ctx->func_attr_mask |= (1ull << cfg_id);
  }
  const int grid = static_cast<int>(p.total_tiles < ctx->num_sms ? p.total_tiles : ctx->num_sms);
  p.step_m = grid % p.tiles_m;
  p.step_n = (grid / p.tiles_m) % p.tiles_n;
  p.step_b = (grid / p.tiles_m) / p.tiles_n;
  ctx->pdl_next_gemm = 0;
  MB_CUDA(ctx, mb_launch_chained(ctx, kern, dim3(grid), dim3(NUM_THREADS), Cfg::SMEM_BYTES, ta, tb, tc, p));
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  ctx->launches_tc++;
  return MB_SUCCESS;
}

// The CTA-pair kernel: clusters of two, as many as there are SM pairs (or tiles).
template <bool A_MN, bool B_MN>
int launch_pair(mb_context *ctx, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc, TcParams &p) {
  using Cfg = TileCfg<256, B_MN, BK, false, true>;
  auto kern = gemm_u8_tc_kernel<256, A_MN, B_MN, false, BK, false, true>;
  constexpr int cfg_id = 56 + (A_MN ? 2 : 0) + (B_MN ? 1 : 0);
  if (!(ctx->func_attr_mask & (1ull << cfg_id))) {
    MB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    ctx->func_attr_mask |= (1ull << cfg_id);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(NUM_THREADS);
  // The tiles are dealt out to the clusters once, so every cluster of the launch has to be
  // resident at the same time: ask how many fit (the SMs of a pair share a TPC, and not every
  // TPC of every GPC need be available), once per context.
  if (ctx->max_pair_clusters == 0) {
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(2 * (ctx->num_sms / 2));
    probe.blockDim = dim3(NUM_THREADS);
    probe.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cudaLaunchAttribute pa[1];
    pa[0].id = cudaLaunchAttributeClusterDimension;
    pa[0].val.clusterDim.x = 2;
    pa[0].val.clusterDim.y = 1;
    pa[0].val.clusterDim.z = 1;
    probe.attrs = pa;
    probe.numAttrs = 1;
    int n = 0;
    MB_CUDA(ctx, cudaOccupancyMaxActiveClusters(&n, kern, &probe));
    if (n < 1) return mb_fail(ctx, MB_RUNTIME_ERROR, "no CTA pair of the GEMM kernel fits the device");
    ctx->max_pair_clusters = n;
  }
  const int64_t pairs = std::min<int64_t>(ctx->num_sms / 2, ctx->max_pair_clusters);
  const int clusters = static_cast<int>(p.total_tiles < pairs ? p.total_tiles : pairs);
  p.step_m = clusters % p.tiles_m;
  p.step_n = (clusters / p.tiles_m) % p.tiles_n;
  p.step_b = (clusters / p.tiles_m) / p.tiles_n;
  ctx->pdl_next_gemm = 0;
  cfg.gridDim = dim3(2 * clusters);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl_chain ? 2 : 1;
  MB_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, p));
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  ctx->launches_tc++;
  ctx->launches_pair++;
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
static int tc_launch_impl(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                          const uint32_t *sum_a, const uint32_t *sum_b, int sum_a_slices, int sum_b_slices,
                          const int32_t *bias,
                          void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N,
                          int64_t K, bool a_mn, bool b_mn, int a_batched, int b_batched,
                          int32_t zp_a, int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c,
                          int bias_per_row, int float_rule, float mult_f, int add_zp, int k_split = 1,
                          int bn_forced = 0) {
  // k_split > 1: one product whose depth is cut into k_split equal runs, computed as a batch of
  // k_split products (int32 results [k_split][M][N], each with its own zero-point terms, which
  // are linear in the depth); the caller adds them up.
  const int64_t k_full = K;
  if (k_split > 1) {
    K /= k_split;
    batch = k_split;
    a_batched = b_batched = 1;
  }
  // Operand sums computed inside the kernel: K-major operands, short K, and the
  // caller passed no precomputed sums although a zero point needs them.
  // Rows of 64 or 32 bytes for K-major operands with K <= 64 (the first pointwise
  // convolutions of a network): the TMA boxes then hold no out-of-range bytes.  These
  // shapes always take the fused kernel (it also serves zero points of 0).
  const bool kmajor_free = !a_mn && !b_mn && sum_a == nullptr && sum_b == nullptr;
  const int KBsel = (kmajor_free && K <= 32) ? 32 : (kmajor_free && K <= 64) ? 64 : BK;
  const bool fuse = kmajor_free && K <= 8 * BK && (zp_a != 0 || zp_b != 0 || KBsel != BK);
  // a K-major A against a row-major B with a depth (or depth run) of at most 1024: B's column
  // sums are taken from the tiles too, word by word (depth runs are bound by the bytes each SM
  // can pull and short-depth products by their epilogue: the tile readers have the time)
  const bool fuse_bmn = !a_mn && b_mn && sum_a == nullptr && sum_b == nullptr && K <= 8 * BK &&
                        (zp_a != 0 || zp_b != 0);
  // Tile width.  Long main loops (K > 1024) want the widest tile for operand
  // reuse -- unless that leaves most SMs without a tile (a few rows against a
  // large B): then the width with the fewest columns per SM wins, wider on a
  // tie, so that B streams through as many SMs as possible.  Short main loops
  // are bound by the epilogue, whose cost grows with the width, plus a fixed
  // cost per tile: pick the width with the fewest rounds of (width + overhead)
  // over the SMs.
  int BN = 64;
  {
    const int64_t tm = ceil_div64(M, BM);
    const int widths[3] = {256, 128, 64};
    int64_t best = -1;
    bool widest_seen = false, spread = false;
    for (int w : widths) {
      if (w > 64 && N <= w / 2) continue;  // more than half of the tile would be padding
      const int64_t tiles = batch * tm * ceil_div64(N, w);
      const int64_t rounds = ceil_div64(tiles, ctx->num_sms);
      if (K > 1024) {
        if (!widest_seen) {
          widest_seen = true;
          BN = w;
          if (tiles >= ctx->num_sms) break;  // every SM has work at the widest width
          spread = true;
          best = rounds * w;
          continue;
        }
        if (spread && rounds * w < best) {
          best = rounds * w;
          BN = w;
        }
        continue;
      }
      const int64_t cost = rounds * (w + 96);
      if (best < 0 || cost < best) {
        best = cost;
        BN = w;
      }
    }
    if (ctx->force_bn != 0 && !(ctx->force_bn > 64 && N <= ctx->force_bn / 2)) BN = ctx->force_bn;
    if (bn_forced != 0) BN = bn_forced;
  }
  TcParams p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.tiles_m = static_cast<int>(ceil_div64(M, BM));
  p.tiles_n = static_cast<int>(ceil_div64(N, BN));
  p.k_blocks = static_cast<int>(ceil_div64(K, KBsel));
  p.total_tiles = batch * p.tiles_m * p.tiles_n;
  p.sum_a = sum_a; p.sum_b = sum_b;
  p.sum_a_slices = sum_a_slices; p.sum_b_slices = sum_b_slices;
  p.sum_a_bstride = M * sum_a_slices; p.sum_b_bstride = N * sum_b_slices;
  p.a_batched = a_batched; p.b_batched = b_batched;
  p.bias = bias; p.bias_per_row = bias_per_row;
  p.zp_a = zp_a; p.zp_b = zp_b;
  p.rq = mb_make_requant(mult, shift, zp_c);
  p.rq_variant = float_rule ? 8 : mb_requant_variant(shift, zp_c);
  p.mult_f = mult_f;
  p.zp_f = add_zp ? static_cast<float>(zp_c) : 0.f;
  p.kzz = static_cast<int32_t>(static_cast<uint32_t>(K) * static_cast<uint32_t>(zp_a) *
                               static_cast<uint32_t>(zp_b));
  p.C = C; p.out_is_int32 = out_is_int32;
  const uintptr_t cbase = reinterpret_cast<uintptr_t>(C);
  p.c_tma = (!out_is_int32 && cbase % 16 == 0 && N % 16 == 0 && N >= 64 && M >= 32) ? 1 : 0;
  p.status = ctx->dev_status;
  p.timeline = ctx->tc_timeline;
  p.b_const = (ctx->gemm_b_const && ctx->b_prefetch) ? 1 : 0;
  p.sums_pending = (ctx->pdl_next_gemm && ctx->pdl_chain && (sum_a != nullptr || sum_b != nullptr)) ? 1 : 0;
  // At least one round of 256 x 256 tiles over the SM pairs: two CTAs per tile, each loading
  // half of it (the lone-CTA kernel is bound by the bytes its 128 x 256 tiles pull from L2).
  // (option value 2 takes the pair kernel wherever it can run, for tests on small shapes)
  const bool pair = ctx->pair_gemm && !fuse && !fuse_bmn && k_split == 1 && p.c_tma && ctx->num_sms >= 2 &&
                    (ctx->pair_gemm == 2 ||
                     (BN == 256 && K >= 512 && batch * ceil_div64(M, 256) * ceil_div64(N, 256) >= ctx->num_sms / 2));
  if (pair) {
    BN = 256;
    p.tiles_n = static_cast<int>(ceil_div64(N, 256));
    p.tiles_m = static_cast<int>(ceil_div64(M, 256));
    p.total_tiles = batch * p.tiles_m * p.tiles_n;
  }

  CUtensorMap ta, tb, tc;
  if (p.c_tma) {
    // the staged box is 32 bytes wide for 256-wide tiles, else 64 (TileCfg::STG_CHUNKS)
    if (BN == 256) {
      MB_RETURN_IF_ERROR(make_map_u8(ctx, &tc, C, N, M, batch, M * N, 32, 32, CU_TENSOR_MAP_SWIZZLE_32B));
    } else {
      MB_RETURN_IF_ERROR(make_map_u8(ctx, &tc, C, N, M, batch, M * N, 64, 32, CU_TENSOR_MAP_SWIZZLE_64B));
    }
  } else {
    memset(&tc, 0, sizeof(tc));
  }
  const uint64_t nb_a = a_batched ? batch : 1, nb_b = b_batched ? batch : 1;
  const CUtensorMapSwizzle kswz = KBsel == 32   ? CU_TENSOR_MAP_SWIZZLE_32B
                                  : KBsel == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                : CU_TENSOR_MAP_SWIZZLE_128B;
  // (a run of the depth: K-major rows keep the pitch of the whole matrix and the runs lie side by
  // side; MN-major runs are whole row blocks, one behind the other)
  if (a_mn) {
    MB_RETURN_IF_ERROR(make_map_u8(ctx, &ta, A, M, K, nb_a, M * K, 128, BK));
  } else {
    MB_RETURN_IF_ERROR(make_map_u8(ctx, &ta, A, K, M, nb_a, k_split > 1 ? K : M * K, KBsel, BM, kswz, k_full));
  }
  if (b_mn) {
    MB_RETURN_IF_ERROR(make_map_u8(ctx, &tb, B, N, K, nb_b, N * K, 128, BK));
  } else {
    MB_RETURN_IF_ERROR(make_map_u8(ctx, &tb, B, K, N, nb_b, k_split > 1 ? K : N * K, KBsel, pair ? 128 : BN, kswz, k_full));
  }
  if (pair) {
    if (a_mn) {
      if (b_mn) return launch_pair<true, true>(ctx, ta, tb, tc, p);
      return launch_pair<true, false>(ctx, ta, tb, tc, p);
    }
    if (b_mn) return launch_pair<false, true>(ctx, ta, tb, tc, p);
    return launch_pair<false, false>(ctx, ta, tb, tc, p);
  }

#define MB_TC_DISPATCH(BN_)                                                         \
  if (a_mn) {                                                                       \
    if (b_mn) return launch_cfg<BN_, true, true>(ctx, ta, tb, tc, p);                   \
    return launch_cfg<BN_, true, false>(ctx, ta, tb, tc, p);                            \
  } else {                                                                          \
    if (b_mn) return launch_cfg<BN_, false, true>(ctx, ta, tb, tc, p);                  \
    return launch_cfg<BN_, false, false>(ctx, ta, tb, tc, p);                           \
  }
  if (fuse_bmn) {
    if (BN == 256) return launch_cfg<256, false, true, true>(ctx, ta, tb, tc, p);
    if (BN == 128) return launch_cfg<128, false, true, true>(ctx, ta, tb, tc, p);
    return launch_cfg<64, false, true, true>(ctx, ta, tb, tc, p);
  }
  if (fuse) {
#define MB_TC_FUSED(KB_)                                                                  \
  if (BN == 256) return launch_cfg<256, false, false, true, KB_>(ctx, ta, tb, tc, p);     \
  if (ctx->tc_rowsum) {                                                                            \
    if (BN == 128) return launch_cfg<128, false, false, true, KB_, true>(ctx, ta, tb, tc, p); \
    return launch_cfg<64, false, false, true, KB_, true>(ctx, ta, tb, tc, p);             \
  }                                                                                                \
  if (BN == 128) return launch_cfg<128, false, false, true, KB_>(ctx, ta, tb, tc, p);     \
  return launch_cfg<64, false, false, true, KB_>(ctx, ta, tb, tc, p);
    if (KBsel == 32) { MB_TC_FUSED(32) }
    if (KBsel == 64) { MB_TC_FUSED(64) }
    MB_TC_FUSED(128)
#undef MB_TC_FUSED
  }
  if (BN == 256) { MB_TC_DISPATCH(256) }
  if (BN == 128) { MB_TC_DISPATCH(128) }
  MB_TC_DISPATCH(64)
#undef MB_TC_DISPATCH
}

int mb_gemm_u8_tc_launch(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                         const uint32_t *sum_a, const uint32_t *sum_b, const int32_t *bias,
                         void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N,
                         int64_t K, bool a_mn, bool b_mn, int a_batched, int b_batched,
                         int32_t zp_a, int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c,
                         int bias_per_row) {
  return tc_launch_impl(ctx, A, B, sum_a, sum_b, 1, 1, bias, C, out_is_int32, batch, M, N, K, a_mn, b_mn,
                        a_batched, b_batched, zp_a, zp_b, mult, shift, zp_c, bias_per_row, 0, 0.f, 0);
}

// The same with each operand's sums given as `slices` partial rows ([batch or 1][slices][extent]),
// as mb_operand_sums_launch writes the column sums of an MN-major operand.
int mb_gemm_u8_tc_launch_sliced(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                                const uint32_t *sum_a, const uint32_t *sum_b, int sum_a_slices, int sum_b_slices,
                                const int32_t *bias, void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N,
                                int64_t K, bool a_mn, bool b_mn, int a_batched, int b_batched,
                                int32_t zp_a, int32_t zp_b, int32_t mult, int32_t shift, int32_t zp_c,
                                int bias_per_row) {
  return tc_launch_impl(ctx, A, B, sum_a, sum_b, sum_a_slices, sum_b_slices, bias, C, out_is_int32, batch, M, N, K,
                        a_mn, b_mn, a_batched, b_batched, zp_a, zp_b, mult, shift, zp_c, bias_per_row, 0, 0.f, 0);
}

// One product with its depth cut into k_split equal runs (K % (k_split * 128) == 0): `parts`
// receives the k_split int32 results [k_split][M][N], each the exact sum over its run of
// (A - zp_a)(B - zp_b); the sums are per run ([k_split][...], see mb_operand_sums_launch).
int mb_gemm_u8_tc_launch_splitk(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                                const uint32_t *sum_a, const uint32_t *sum_b, int sum_a_slices, int sum_b_slices,
                                int32_t *parts, int k_split, int bn, int64_t M, int64_t N, int64_t K, bool a_mn,
                                bool b_mn, int32_t zp_a, int32_t zp_b) {
  return tc_launch_impl(ctx, A, B, sum_a, sum_b, sum_a_slices, sum_b_slices, nullptr, parts, 1, 1, M, N, K, a_mn,
                        b_mn, 0, 0, zp_a, zp_b, 1 << 30, 0, 0, 0, 0, 0.f, 0, k_split, bn);
}

// The same product with the Gemv delegators' float requantization rule (see
// requant_float_rule): K-major operands, operand sums taken inside the kernel.
int mb_gemm_u8_tc_launch_float_rule(mb_context *ctx, const uint8_t *A, const uint8_t *B,
                                    const int32_t *bias, void *C, int out_is_int32, int64_t M,
                                    int64_t N, int64_t K, int32_t zp_a, int32_t zp_b, float mult_f,
                                    int32_t zp_c, int add_zp) {
  return tc_launch_impl(ctx, A, B, nullptr, nullptr, 1, 1, bias, C, out_is_int32, 1, M, N, K, false, false, 0,
                        0, zp_a, zp_b, 1 << 30, 0, zp_c, 0, 1, mult_f, add_zp);
}
