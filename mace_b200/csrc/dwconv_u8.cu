// uint8 depthwise convolution, NHWC input, HWIM filter, NHWC output.
//
// Reference behaviour: DepthwiseConv2dOp<RT_CPU,uint8_t>::Run
// (mace/ops/depthwise_conv2d.cc:152-250): int32 accumulation of
// (in - zp_in) * (f - zp_f) over the taps that fall inside the image, + bias,
// fixed-point requantization (same primitives as the GEMM output pipeline),
// + zp_out, clamp to [0,255]; and its dilated fallback DepthwiseConv2dGeneral
// (:252-320), which requantizes with int(round(acc * multiplier_float)).
//
// Data layout: channels are innermost, so one warp reads 128 consecutive
// channel bytes of a pixel in one transaction.  Each thread owns 4 adjacent
// channels (one 32-bit word per tap) and a short strip of output pixels along
// W; the filter taps of its channels stay in registers for the whole strip.
#include <algorithm>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

struct DwParams {
  const uint8_t *in, *filter;
  const int32_t *bias;
  uint8_t *out;
  int N, H, W, C, mult_ch, KH, KW, stride_h, stride_w, dil_h, dil_w, pad_top, pad_left, Ho, Wo;
  int32_t zp_in, zp_f, zp_out;
  mb_requant_params rq;
  int use_float;
  float mult_f;
};

__device__ __forceinline__ uint32_t dw_requant(int32_t acc, const DwParams &p) {
  if (p.use_float) {
    // sum = static_cast<int32_t>(std::round(sum * multiplier)); sum += zp_out
    const int32_t v =
        static_cast<int32_t>(roundf(__fmul_rn(static_cast<float>(acc), p.mult_f))) + p.zp_out;
    return static_cast<uint32_t>(min(255, max(0, v)));
  }
  return mb_requant_fast(acc, p.rq);
}

// ---- fast path: 3x3, channel multiplier 1, dilation 1, stride 1 or 2, C % 4 == 0 -------
//
// Arithmetic.  With raw input bytes and w = f - zp_f:
//   sum (in - zp_in) w = sum in * w - zp_in * sum w,
// out-of-image taps read as zp_in (they then contribute zero).  dp4a multiplies four
// unsigned input bytes with four SIGNED 8-bit weights, but w needs 9 bits.  It is split as
// w = w1 + w2 with w1 = clamp(w, -128, 127): w2 is zero except for the few taps at the far
// end of the filter's range (none at all when zp_f == 128), and channel groups that have
// such a tap run a second dp4a with w2.
//
// Layout of the work.  A thread owns 4 adjacent channels (one 32-bit word per pixel), 4
// adjacent output columns and a run of output rows.  Per input row it loads the 6 (stride
// 1) or 9 (stride 2) pixel words its columns touch and transposes them with byte permutes
// into per-channel words of 4 horizontally adjacent pixels ("windows"), so that ONE dp4a
// covers the three taps of a filter row: stride 1 uses window [x-1,x,x+1,x+2] for output x
// (weights [w0,w1,w2,0]) and for output x+1 (weights [0,w0,w1,w2]).  Every input row is
// loaded and transposed once and used for the three output rows it belongs to.
//
// The prepack kernel turns the HWIM filter (+ bias) into those weight words once per call
// (or once per weight tensor through mb_dwconv_u8_prepack).

// Per group of 4 channels, as structure of arrays [item][group] of 16-byte items:
//   0..5   w1[kh][align] : x,y,z,w = channels; bytes = [w0,w1,w2,0] (align 0) / [0,w0,w1,w2]
//   6..11  w2[kh][align]
//   12     start[c] = bias[c] - zp_in * sum_t w[t][c]
//   13     flags: x = group has a non-zero w2; y = bit kh set when filter row kh has one
constexpr int DW_PACK_ITEMS = 14;
#ifndef DW_THREADS
#define DW_THREADS 256
#define DW_BLOCKS_PER_SM 2
#endif

__device__ __forceinline__ int32_t dp4a_u8_s8(uint32_t a, uint32_t b, int32_t c) {
  int32_t d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

__global__ void __launch_bounds__(128)
dwconv3x3_prepack_kernel(const uint8_t *__restrict__ filter, const int32_t *__restrict__ bias,
                         uint4 *__restrict__ packed, int C, int32_t zp_in, int32_t zp_f) {
  const int groups = C >> 2;
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  int32_t w[9][4];
#pragma unroll
  for (int t = 0; t < 9; ++t) {
    const uint32_t v = __ldg(reinterpret_cast<const uint32_t *>(filter + t * C + g * 4));
#pragma unroll
    for (int c = 0; c < 4; ++c) w[t][c] = static_cast<int32_t>((v >> (8 * c)) & 0xffu) - zp_f;
  }
  int32_t any_w2 = 0;
  uint32_t rows_w2 = 0;
  uint32_t v1[3][2][4], v2[3][2][4];
  int32_t start[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    int32_t sum = 0;
#pragma unroll
    for (int kh = 0; kh < 3; ++kh) {
      uint32_t p1 = 0, p2 = 0;
#pragma unroll
      for (int kw = 0; kw < 3; ++kw) {
        const int32_t x = w[kh * 3 + kw][c];
        const int32_t a = min(127, max(-128, x)), b = x - a;
        sum += x;
        any_w2 |= b;
        if (b != 0) rows_w2 |= 1u << kh;
        p1 |= (static_cast<uint32_t>(a) & 0xffu) << (8 * kw);
        p2 |= (static_cast<uint32_t>(b) & 0xffu) << (8 * kw);
      }
      v1[kh][0][c] = p1; v1[kh][1][c] = p1 << 8;
      v2[kh][0][c] = p2; v2[kh][1][c] = p2 << 8;
    }
    const int32_t bv = bias != nullptr ? __ldg(bias + g * 4 + c) : 0;
    start[c] = bv - zp_in * sum;
  }
#pragma unroll
  for (int kh = 0; kh < 3; ++kh)
#pragma unroll
    for (int al = 0; al < 2; ++al) {
      packed[(kh * 2 + al) * groups + g] =
          make_uint4(v1[kh][al][0], v1[kh][al][1], v1[kh][al][2], v1[kh][al][3]);
      packed[(6 + kh * 2 + al) * groups + g] =
          make_uint4(v2[kh][al][0], v2[kh][al][1], v2[kh][al][2], v2[kh][al][3]);
    }
  packed[12 * groups + g] = make_uint4(start[0], start[1], start[2], start[3]);
  packed[13 * groups + g] = make_uint4(any_w2 != 0 ? 1u : 0u, rows_w2, 0u, 0u);
}

// Windows of one input row: win[j][c] holds, for channel c, the 4 horizontally adjacent
// input bytes that output column j / pair of columns needs (see the kernel).
template <int STRIDE>
struct DwRow {
  // stride 1: win[0] = cols 0..3, win[1] = cols 2..5  (relative to the strip's first column)
  // stride 2: win[j] = cols 2j .. 2j+3, j = 0..3
  uint32_t win[STRIDE == 1 ? 2 : 4][4];
};

template <int STRIDE>
struct DwRaw {
  uint32_t q[STRIDE == 1 ? 6 : 9];
};

// Loads the pixel words of one input row.  Addresses are a uniform base plus an unsigned
// 32-bit offset (the host keeps the fast path to tensors below 4 GB), which keeps the
// per-load address arithmetic to one 32-bit addition.
template <int STRIDE>
__device__ __forceinline__ void dw_load_raw(DwRaw<STRIDE> &raw, const uint8_t *__restrict__ in,
                                            uint32_t thread_off, int hi, int H, uint32_t row_stride,
                                            const uint32_t (&col_off)[STRIDE == 1 ? 6 : 9],
                                            uint32_t col_ok, uint32_t zi4) {
  constexpr int COLS = STRIDE == 1 ? 6 : 9;
  constexpr uint32_t ALL = (1u << COLS) - 1u;
  if (hi < 0 || hi >= H) {  // a row outside the image reads as the input zero point
#pragma unroll
    for (int j = 0; j < COLS; ++j) raw.q[j] = zi4;
    return;
  }
  const uint32_t row_off = thread_off + static_cast<uint32_t>(hi) * row_stride;
  if (col_ok == ALL) {
#pragma unroll
    for (int j = 0; j < COLS; ++j)
      raw.q[j] = __ldg(reinterpret_cast<const uint32_t *>(in + (row_off + col_off[j])));
  } else {
#pragma unroll
    for (int j = 0; j < COLS; ++j)
      raw.q[j] = ((col_ok >> j) & 1u) ? __ldg(reinterpret_cast<const uint32_t *>(in + (row_off + col_off[j]))) : zi4;
  }
}

template <int STRIDE>
__device__ __forceinline__ void dw_transpose(const DwRaw<STRIDE> &raw, DwRow<STRIDE> &row) {
  // pair stage: lo = [a.b0, b.b0, a.b1, b.b1], hi = [a.b2, b.b2, a.b3, b.b3]
  constexpr int PAIRS = STRIDE == 1 ? 3 : 4;
  uint32_t lo[PAIRS], hi[PAIRS];
#pragma unroll
  for (int k = 0; k < PAIRS; ++k) {
    lo[k] = __byte_perm(raw.q[2 * k], raw.q[2 * k + 1], 0x5140);
    hi[k] = __byte_perm(raw.q[2 * k], raw.q[2 * k + 1], 0x7362);
  }
  constexpr int FULL = STRIDE == 1 ? 2 : 3;  // windows made of two pairs
#pragma unroll
  for (int j = 0; j < FULL; ++j) {
    row.win[j][0] = __byte_perm(lo[j], lo[j + 1], 0x5410);
    row.win[j][1] = __byte_perm(lo[j], lo[j + 1], 0x7632);
    row.win[j][2] = __byte_perm(hi[j], hi[j + 1], 0x5410);
    row.win[j][3] = __byte_perm(hi[j], hi[j + 1], 0x7632);
  }
  if constexpr (STRIDE == 2) {  // last window: cols 6, 7 from the last pair, col 8 from its own word
    const uint32_t q8 = raw.q[8];
    row.win[FULL][0] = __byte_perm(lo[PAIRS - 1], q8, 0x4410);
    row.win[FULL][1] = __byte_perm(lo[PAIRS - 1], q8, 0x5532);
    row.win[FULL][2] = __byte_perm(hi[PAIRS - 1], q8, 0x6610);
    row.win[FULL][3] = __byte_perm(hi[PAIRS - 1], q8, 0x7732);
  }
}

// acc[j][c] += one filter row (weights wa = [w0,w1,w2,0], wb = [0,w0,w1,w2]) times the row.
template <int STRIDE>
__device__ __forceinline__ void dw_mac(int32_t (&acc)[4][4], const DwRow<STRIDE> &row, const uint4 wa,
                                       const uint4 wb) {
  const uint32_t a[4] = {wa.x, wa.y, wa.z, wa.w};
  const uint32_t b[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    if constexpr (STRIDE == 1) {
      acc[0][c] = dp4a_u8_s8(row.win[0][c], a[c], acc[0][c]);
      acc[1][c] = dp4a_u8_s8(row.win[0][c], b[c], acc[1][c]);
      acc[2][c] = dp4a_u8_s8(row.win[1][c], a[c], acc[2][c]);
      acc[3][c] = dp4a_u8_s8(row.win[1][c], b[c], acc[3][c]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[j][c] = dp4a_u8_s8(row.win[j][c], a[c], acc[j][c]);
    }
  }
}

// VAR: requantization variant (mb_requant_variant): 0..3 = mb_requant_t, 4 / 5 = packed form.
template <int STRIDE, int VAR>
__global__ void __launch_bounds__(DW_THREADS, DW_BLOCKS_PER_SM)
dwconv3x3_u8_kernel(const DwParams p, const uint4 *__restrict__ packed, int rows_per_thread,
                    int segments, int weights_cached) {
  constexpr int COLS = STRIDE == 1 ? 6 : 9;
  mb_grid_dep_launch();
  // weights_cached: the tap words were complete before the kernel in front of this one started
  // (the host checks that the prepack kernel is not that kernel), so they may be fetched before
  // the wait for the previous kernel, whose output is this kernel's input.  Otherwise only the
  // wait makes the predecessor's writes visible.
  if (!weights_cached) mb_grid_dep_wait();
  const int groups = p.C >> 2;
  const int strips = (p.Wo + 3) >> 2;
  const int per_seg = groups * strips;
  const unsigned per_image = static_cast<unsigned>(per_seg) * segments;
  const unsigned id = blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned n = id / per_image;
  if (n >= static_cast<unsigned>(p.N)) return;
  const int rem_n = id - n * per_image;
  const int seg = rem_n / per_seg;
  const int rem = rem_n - seg * per_seg;
  const int strip = rem / groups;
  const int g = rem - strip * groups;
  const int y0 = seg * rows_per_thread;
  const int y1 = min(p.Ho, y0 + rows_per_thread);
  if (y0 >= y1) return;
  const int x0 = strip * 4;

  uint4 w1[3][2];
#pragma unroll
  for (int kh = 0; kh < 3; ++kh) {
    w1[kh][0] = __ldg(packed + (kh * 2 + 0) * groups + g);
    if (STRIDE == 1) w1[kh][1] = __ldg(packed + (kh * 2 + 1) * groups + g);
    else w1[kh][1] = w1[kh][0];
  }
  const uint4 st4 = __ldg(packed + 12 * groups + g);
  const uint4 flags = __ldg(packed + 13 * groups + g);
  const int32_t start[4] = {static_cast<int32_t>(st4.x), static_cast<int32_t>(st4.y),
                            static_cast<int32_t>(st4.z), static_cast<int32_t>(st4.w)};
  const bool has_w2 = flags.x != 0;
  const uint32_t rows_w2 = flags.y;  // the filter rows that have a 9-bit tap (rare: most warps skip most rows)
  if (weights_cached) mb_grid_dep_wait();

  // columns: byte offsets inside a row and validity bits, fixed for the thread
  uint32_t col_off[COLS];
  uint32_t col_ok = 0;
  const int xi0 = x0 * STRIDE - p.pad_left;
#pragma unroll
  for (int j = 0; j < COLS; ++j) {
    const int xi = xi0 + j;
    const bool ok = xi >= 0 && xi < p.W;
    col_off[j] = static_cast<uint32_t>(ok ? xi : 0) * static_cast<uint32_t>(p.C);
    col_ok |= ok ? (1u << j) : 0u;
  }
  const uint32_t zi4 = static_cast<uint32_t>(p.zp_in) * 0x01010101u;
  const uint32_t row_stride = static_cast<uint32_t>(p.W) * p.C;
  const uint32_t in_off = n * static_cast<uint32_t>(p.H) * row_stride + g * 4;
  const uint32_t out_row_stride = static_cast<uint32_t>(p.Wo) * p.C;
  const uint32_t out_off = n * static_cast<uint32_t>(p.Ho) * out_row_stride + g * 4 +
                           static_cast<uint32_t>(x0) * p.C;
  const uint8_t *__restrict__ in = p.in;
  uint8_t *__restrict__ out = p.out;
  const int valid_cols = min(4, p.Wo - x0);

  // one output row from three input rows
  auto emit = [&](int y, const DwRow<STRIDE> &r0, const DwRow<STRIDE> &r1, const DwRow<STRIDE> &r2) {
    int32_t acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[j][c] = start[c];
    dw_mac<STRIDE>(acc, r0, w1[0][0], w1[0][1]);
    dw_mac<STRIDE>(acc, r1, w1[1][0], w1[1][1]);
    dw_mac<STRIDE>(acc, r2, w1[2][0], w1[2][1]);
    if (has_w2) {
      if (rows_w2 & 1u) dw_mac<STRIDE>(acc, r0, __ldg(packed + 6 * groups + g), __ldg(packed + 7 * groups + g));
      if (rows_w2 & 2u) dw_mac<STRIDE>(acc, r1, __ldg(packed + 8 * groups + g), __ldg(packed + 9 * groups + g));
      if (rows_w2 & 4u) dw_mac<STRIDE>(acc, r2, __ldg(packed + 10 * groups + g), __ldg(packed + 11 * groups + g));
    }
    uint32_t o = out_off + static_cast<uint32_t>(y) * out_row_stride;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t word;
      if (VAR >= 4) {
        word = mb_requant_pack4<VAR == 5>(acc[j][0], acc[j][1], acc[j][2], acc[j][3], p.rq);
      } else {
        uint32_t b[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) b[c] = mb_requant_t<(VAR & 1) != 0, (VAR & 2) != 0>(acc[j][c], p.rq);
        word = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
      }
      if (j < valid_cols) *reinterpret_cast<uint32_t *>(out + o) = word;
      o += p.C;
    }
  };

  DwRaw<STRIDE> raw;
  DwRow<STRIDE> ra, rb, rc;
  const int hi0 = y0 * STRIDE - p.pad_top;
  if constexpr (STRIDE == 1) {
    // rows hi0, hi0+1 first; then one new input row per output row, requested one output
    // row ahead of its use so that the load is in flight during the arithmetic
    dw_load_raw<STRIDE>(raw, in, in_off, hi0, p.H, row_stride, col_off, col_ok, zi4);
    dw_transpose<STRIDE>(raw, ra);
    dw_load_raw<STRIDE>(raw, in, in_off, hi0 + 1, p.H, row_stride, col_off, col_ok, zi4);
    dw_transpose<STRIDE>(raw, rb);
    dw_load_raw<STRIDE>(raw, in, in_off, hi0 + 2, p.H, row_stride, col_off, col_ok, zi4);
    for (int y = y0; y < y1; y += 3) {
      dw_transpose<STRIDE>(raw, rc);
      dw_load_raw<STRIDE>(raw, in, in_off, y - p.pad_top + 3, p.H, row_stride, col_off, col_ok, zi4);
      emit(y, ra, rb, rc);
      if (y + 1 < y1) {
        dw_transpose<STRIDE>(raw, ra);
        dw_load_raw<STRIDE>(raw, in, in_off, y - p.pad_top + 4, p.H, row_stride, col_off, col_ok, zi4);
        emit(y + 1, rb, rc, ra);
      }
      if (y + 2 < y1) {
        dw_transpose<STRIDE>(raw, rb);
        dw_load_raw<STRIDE>(raw, in, in_off, y - p.pad_top + 5, p.H, row_stride, col_off, col_ok, zi4);
        emit(y + 2, rc, ra, rb);
      }
    }
  } else {
    // output row y reads input rows 2y-pad .. 2y-pad+2; the last one is the next row's first
    dw_load_raw<STRIDE>(raw, in, in_off, hi0, p.H, row_stride, col_off, col_ok, zi4);
    dw_transpose<STRIDE>(raw, ra);
    for (int y = y0; y < y1; y += 2) {
      const int hi = y * 2 - p.pad_top;
      dw_load_raw<STRIDE>(raw, in, in_off, hi + 1, p.H, row_stride, col_off, col_ok, zi4);
      dw_transpose<STRIDE>(raw, rb);
      dw_load_raw<STRIDE>(raw, in, in_off, hi + 2, p.H, row_stride, col_off, col_ok, zi4);
      dw_transpose<STRIDE>(raw, rc);
      emit(y, ra, rb, rc);
      if (y + 1 < y1) {
        dw_load_raw<STRIDE>(raw, in, in_off, hi + 3, p.H, row_stride, col_off, col_ok, zi4);
        dw_transpose<STRIDE>(raw, rb);
        dw_load_raw<STRIDE>(raw, in, in_off, hi + 4, p.H, row_stride, col_off, col_ok, zi4);
        dw_transpose<STRIDE>(raw, ra);
        emit(y + 1, rc, rb, ra);
      }
    }
  }
}

// ---- the same arithmetic fed from shared memory by TMA ------------------------------------------
//
// A CTA owns one image, a run of output rows, a tile of output columns and a chunk of CB
// channel bytes.  Thread 0 asks for every input row the run needs at once -- one tiled TMA copy
// per row, a box of [TWB columns x CB channels] with its own mbarrier -- so the whole tile
// (up to ~70 KB) is in flight while the threads work on the rows that have landed; columns and
// rows outside the image arrive as zeros, which is the input zero point of the tensors this
// path takes (activations behind a ReLU; other zero points use the register kernel above), so
// no thread tests a boundary.  The compute is the register kernel's: a thread owns 4 channels
// x 4 output columns, reads the 6 (stride 1) or 9 (stride 2) pixel words of a new input row
// from shared memory, transposes them into 4-pixel windows and multiplies with dp4a; two
// earlier rows stay in registers.
struct DwTmaTile {
  int CB, G;          // channel bytes / channel groups (of 4) per CTA
  int strips, OWT;    // 4-column strips and output columns per tile (OWT = 4 * strips)
  int TWB;            // input columns per row box
  int row_pitch;      // bytes between rows in shared memory (TMA wants 128-byte aligned targets)
  int rows_out;       // output rows per CTA
  int col_tiles, chan_chunks, segments;
  int ring_bytes;     // shared memory for the rows (then one mbarrier per row)
  int setup_lanes;    // threads that share the per-row set-up (barrier, copy request): 32, or 1
  int *status;
};
constexpr long long DW_WAIT_BUDGET = 1ll << 31;

// GT: the number of channel groups per CTA when it is fixed at compile time (8, 16, 32, 64: the
// pixel words of a row are then read at constant offsets from one address), 0 = from the tile.
template <int STRIDE, int VAR, int GT = 0>
__global__ void __launch_bounds__(DW_THREADS, DW_BLOCKS_PER_SM)
dwconv3x3_u8_tma_kernel(const __grid_constant__ CUtensorMap tmap_in, const DwParams p,
                        const uint4 *__restrict__ packed, const DwTmaTile t, int weights_cached) {
  extern __shared__ uint8_t dw_smem_raw[];
  __shared__ int abort_flag;
  constexpr int COLS = STRIDE == 1 ? 6 : 9;
  mb_grid_dep_launch();
  // TMA targets must be 128-byte aligned
  uint8_t *dw_smem = dw_smem_raw + ((128u - (sm100::smem_u32(dw_smem_raw) & 127u)) & 127u);
  uint64_t *bars = reinterpret_cast<uint64_t *>(dw_smem + t.ring_bytes);
  unsigned bid = blockIdx.x;
  const int cc = bid % t.chan_chunks; bid /= t.chan_chunks;
  const int ct = bid % t.col_tiles; bid /= t.col_tiles;
  const int seg = bid % t.segments;
  const int n = bid / t.segments;
  const int y0 = seg * t.rows_out;
  const int y1 = min(p.Ho, y0 + t.rows_out);
  const int hi0 = y0 * STRIDE - p.pad_top;           // first input row of the run
  const int rows_in = (y1 - y0 - 1) * STRIDE + 3;
  const int row_bytes = t.TWB * t.CB;
  // (the first warp shares the per-row set-up: a lane per input row)
  if (threadIdx.x < 32) {
    if (threadIdx.x == 0) {
      sm100::prefetch_tensormap(&tmap_in);
      abort_flag = 0;
    }
    if (threadIdx.x < t.setup_lanes)
      for (int r = threadIdx.x; r < rows_in; r += t.setup_lanes) sm100::mbar_init(sm100::smem_u32(bars + r), 1);
    sm100::fence_barrier_init();
  }
  __syncthreads();
  const int G = GT != 0 ? GT : t.G;
  const int g = threadIdx.x % G, strip = threadIdx.x / G;
  const int groups = p.C >> 2;
  const int gg = cc * G + g;  // channel group in the tensor
  if (!weights_cached) mb_grid_dep_wait();
  uint4 w1[3][2];
#pragma unroll
  for (int kh = 0; kh < 3; ++kh) {
    w1[kh][0] = __ldg(packed + (kh * 2 + 0) * groups + gg);
    if (STRIDE == 1) w1[kh][1] = __ldg(packed + (kh * 2 + 1) * groups + gg);
    else w1[kh][1] = w1[kh][0];
  }
  const uint4 st4 = __ldg(packed + 12 * groups + gg);
  const uint4 flags = __ldg(packed + 13 * groups + gg);
  const int32_t start[4] = {static_cast<int32_t>(st4.x), static_cast<int32_t>(st4.y),
                            static_cast<int32_t>(st4.z), static_cast<int32_t>(st4.w)};
  // the filter rows that have a 9-bit tap in ANY lane's channel group (rare: most warps skip most
  // rows); the same for all lanes, so that the tests below do not diverge -- groups without such a
  // tap hold zeros in those weight words
  const uint32_t rows_w2 = __reduce_or_sync(0xffffffffu, flags.x != 0 ? flags.y : 0u);
  if (weights_cached) mb_grid_dep_wait();
  if (threadIdx.x < t.setup_lanes) {
    const int xi0 = ct * t.OWT * STRIDE - p.pad_left;
    for (int r = threadIdx.x; r < rows_in; r += t.setup_lanes) {
      const uint32_t bar = sm100::smem_u32(bars + r);
      sm100::mbar_arrive_expect_tx(bar, static_cast<uint32_t>(row_bytes));
      sm100::tma_load_4d(sm100::smem_u32(dw_smem + r * t.row_pitch), &tmap_in, bar, cc * t.CB, xi0, hi0 + r, n);
    }
  }
  const int x0 = ct * t.OWT + strip * 4;
  if (strip >= t.strips || x0 >= p.Wo) return;  // (no CTA-wide barrier follows)
  const int valid_cols = min(4, p.Wo - x0);
  const uint32_t out_row_stride = static_cast<uint32_t>(p.Wo) * p.C;
  const uint32_t out_off = static_cast<uint32_t>(n) * static_cast<uint32_t>(p.Ho) * out_row_stride + gg * 4 +
                           static_cast<uint32_t>(x0) * p.C;
  uint8_t *__restrict__ out = p.out;
  const uint32_t *sm32 = reinterpret_cast<const uint32_t *>(dw_smem);
  const int row_words = t.row_pitch >> 2;
  const int thread_word = strip * 4 * STRIDE * G + g;  // this thread's first pixel word inside a row
  bool ok = true;

  // the pixel words of input row r of the run (r = 0 is input row hi0), once they have landed
  auto read_row = [&](int r, DwRaw<STRIDE> &raw) {
    if (!sm100::mbar_wait(sm100::smem_u32(bars + r), 0, &abort_flag, DW_WAIT_BUDGET)) {
      abort_flag = 1;
      atomicCAS(t.status, 0, MB_DEV_TIMEOUT_PRODUCER);
      ok = false;
    }
    const uint32_t *w = sm32 + r * row_words + thread_word;
#pragma unroll
    for (int j = 0; j < COLS; ++j) raw.q[j] = w[j * G];
  };
  auto emit = [&](int y, const DwRow<STRIDE> &r0, const DwRow<STRIDE> &r1, const DwRow<STRIDE> &r2) {
    int32_t acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[j][c] = start[c];
    dw_mac<STRIDE>(acc, r0, w1[0][0], w1[0][1]);
    dw_mac<STRIDE>(acc, r1, w1[1][0], w1[1][1]);
    dw_mac<STRIDE>(acc, r2, w1[2][0], w1[2][1]);
    if (rows_w2 & 1u) dw_mac<STRIDE>(acc, r0, __ldg(packed + 6 * groups + gg), __ldg(packed + 7 * groups + gg));
    if (rows_w2 & 2u) dw_mac<STRIDE>(acc, r1, __ldg(packed + 8 * groups + gg), __ldg(packed + 9 * groups + gg));
    if (rows_w2 & 4u) dw_mac<STRIDE>(acc, r2, __ldg(packed + 10 * groups + gg), __ldg(packed + 11 * groups + gg));
    uint32_t o = out_off + static_cast<uint32_t>(y) * out_row_stride;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t word;
      if (VAR >= 4) {
        word = mb_requant_pack4<VAR == 5>(acc[j][0], acc[j][1], acc[j][2], acc[j][3], p.rq);
      } else {
        uint32_t b[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) b[c] = mb_requant_t<(VAR & 1) != 0, (VAR & 2) != 0>(acc[j][c], p.rq);
        word = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
      }
      if (j < valid_cols) *reinterpret_cast<uint32_t *>(out + o) = word;
      o += p.C;
    }
  };

  DwRaw<STRIDE> raw;
  DwRow<STRIDE> ra, rb, rc;
  if constexpr (STRIDE == 1) {
    read_row(0, raw);
    dw_transpose<STRIDE>(raw, ra);
    read_row(1, raw);
    dw_transpose<STRIDE>(raw, rb);
    for (int y = y0; y < y1 && ok; y += 3) {
      const int r = y - y0 + 2;  // run-relative index of the output row's last input row
      read_row(r, raw);
      dw_transpose<STRIDE>(raw, rc);
      emit(y, ra, rb, rc);
      if (y + 1 < y1) {
        read_row(r + 1, raw);
        dw_transpose<STRIDE>(raw, ra);
        emit(y + 1, rb, rc, ra);
      }
      if (y + 2 < y1) {
        read_row(r + 2, raw);
        dw_transpose<STRIDE>(raw, rb);
        emit(y + 2, rc, ra, rb);
      }
    }
  } else {
    read_row(0, raw);
    dw_transpose<STRIDE>(raw, ra);
    for (int y = y0; y < y1 && ok; y += 2) {
      const int r = (y - y0) * 2;
      read_row(r + 1, raw);
      dw_transpose<STRIDE>(raw, rb);
      read_row(r + 2, raw);
      dw_transpose<STRIDE>(raw, rc);
      emit(y, ra, rb, rc);
      if (y + 1 < y1) {
        read_row(r + 3, raw);
        dw_transpose<STRIDE>(raw, rb);
        read_row(r + 4, raw);
        dw_transpose<STRIDE>(raw, ra);
        emit(y + 1, rc, rb, ra);
      }
    }
  }
  // a thread that gave up may leave copies in flight into this CTA's shared memory: let them land
  if (!ok)
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
}

// General path: any filter size, stride, dilation, channel multiplier and
// channel count; one thread per output element.
__global__ void __launch_bounds__(256) dwconv_u8_general_kernel(const DwParams p) {
  const int OC = p.C * p.mult_ch;
  const int64_t total = static_cast<int64_t>(p.N) * p.Ho * p.Wo * OC;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= total) return;
  const int m = static_cast<int>(tid % OC);
  int64_t r = tid / OC;
  const int wo = static_cast<int>(r % p.Wo);
  r /= p.Wo;
  const int ho = static_cast<int>(r % p.Ho);
  const int n = static_cast<int>(r / p.Ho);
  const int c = m / p.mult_ch, o = m % p.mult_ch;
  int32_t acc = 0;
  for (int kh = 0; kh < p.KH; ++kh) {
    const int hi = ho * p.stride_h - p.pad_top + kh * p.dil_h;
    if (hi < 0 || hi >= p.H) continue;
    for (int kw = 0; kw < p.KW; ++kw) {
      const int wi = wo * p.stride_w - p.pad_left + kw * p.dil_w;
      if (wi < 0 || wi >= p.W) continue;
      const int32_t iv = p.in[((static_cast<int64_t>(n) * p.H + hi) * p.W + wi) * p.C + c];
      const int32_t fv = p.filter[((kh * p.KW + kw) * p.C + c) * p.mult_ch + o];
      acc += (iv - p.zp_in) * (fv - p.zp_f);
    }
  }
  if (p.bias != nullptr) acc += p.bias[m];
  p.out[tid] = static_cast<uint8_t>(dw_requant(acc, p));
}

}  // namespace

static int dwconv_u8_impl(mb_context *ctx, const uint8_t *in, const uint8_t *filter,
                                 const int32_t *bias, const void *prepacked, uint8_t *out, int64_t N, int64_t H,
                                 int64_t W, int64_t C, int64_t mult_ch, int64_t KH, int64_t KW,
                                 int stride_h, int stride_w, int dil_h, int dil_w, int pad_top,
                                 int pad_left, int64_t Ho, int64_t Wo, int32_t zp_in,
                                 int32_t zp_f, int32_t multiplier, int32_t right_shift,
                                 int32_t zp_out, int use_float_multiplier, float multiplier_f) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (N < 0 || H < 1 || W < 1 || C < 1 || mult_ch < 1 || KH < 1 || KW < 1 || Ho < 0 || Wo < 0 ||
      stride_h < 1 || stride_w < 1 || dil_h < 1 || dil_w < 1 || pad_top < 0 || pad_left < 0)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_dwconv_u8_nhwc: bad shape argument");
  if (N == 0 || Ho == 0 || Wo == 0) return MB_SUCCESS;
  if (in == nullptr || filter == nullptr || out == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_dwconv_u8_nhwc: null operand");
  if (!use_float_multiplier && (multiplier <= 0 || right_shift < 0 || right_shift > 31))
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_dwconv_u8_nhwc: bad multiplier/shift");
  if (zp_out < 0 || zp_out > 255)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_dwconv_u8_nhwc: output zero point outside uint8");
  if (N * H * W * C >= (1ll << 40) || H > 65535 * 16 || W > 65535 * 16 || C > (1 << 24))
    return mb_fail(ctx, MB_UNSUPPORTED, "mb_dwconv_u8_nhwc: tensor too large");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  DwParams p;
  p.in = in; p.filter = filter; p.bias = bias; p.out = out;
  p.N = static_cast<int>(N); p.H = static_cast<int>(H); p.W = static_cast<int>(W);
  p.C = static_cast<int>(C); p.mult_ch = static_cast<int>(mult_ch);
  p.KH = static_cast<int>(KH); p.KW = static_cast<int>(KW);
  p.stride_h = stride_h; p.stride_w = stride_w; p.dil_h = dil_h; p.dil_w = dil_w;
  p.pad_top = pad_top; p.pad_left = pad_left; p.Ho = static_cast<int>(Ho); p.Wo = static_cast<int>(Wo);
  p.zp_in = zp_in; p.zp_f = zp_f; p.zp_out = zp_out;
  p.rq = mb_make_requant(use_float_multiplier ? (1 << 30) : multiplier, use_float_multiplier ? 0 : right_shift, zp_out);
  p.use_float = use_float_multiplier; p.mult_f = multiplier_f;

  const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(filter) |
                         reinterpret_cast<uintptr_t>(out)) & 3u) == 0;
  const bool fast = KH == 3 && KW == 3 && mult_ch == 1 && dil_h == 1 && dil_w == 1 &&
                    zp_in >= 0 && zp_in <= 255 && zp_f >= 0 && zp_f <= 255 && !use_float_multiplier &&
                    stride_h == stride_w && (stride_h == 1 || stride_h == 2) && C % 4 == 0 &&
                    aligned && N * H * W * C < (1ll << 32) && N * Ho * Wo * C < (1ll << 32) &&
                    (C / 4) * ceil_div64(Wo, 4) * Ho * N < (1ll << 31) - 256;
  if (fast) {
    const int64_t groups = C / 4;
    const uint4 *packed = static_cast<const uint4 *>(prepacked);
    // A caller's tap words may be read ahead of the wait for the previous kernel only when the
    // kernel that wrote them is not that previous kernel: after a (re)pack through this context
    // at least one other kernel must have been launched.  (A copy into the buffer is a full
    // barrier in the stream and needs no care.)
    const int weights_cached = (packed != nullptr && ctx->launches != ctx->dw_prepack_mark) ? 1 : 0;
    if (packed == nullptr) {  // no cached copy: prepare the weight words in scratch
      uint4 *fresh = nullptr;
      MB_RETURN_IF_ERROR(mb_scratch(ctx, sizeof(uint4) * DW_PACK_ITEMS * groups,
                                    reinterpret_cast<void **>(&fresh)));
      dwconv3x3_prepack_kernel<<<static_cast<unsigned>(ceil_div64(groups, 128)), 128, 0, ctx->stream>>>(
          filter, bias, fresh, static_cast<int>(C), zp_in, zp_f);
      MB_CUDA(ctx, cudaGetLastError());
      ctx->launches++;
      packed = fresh;
    }
    // Tensors whose out-of-image taps read as zero (input zero point 0, the activations behind a
    // ReLU) with channel counts TMA can address: rows are fed through shared memory by TMA.
    if (ctx->dw_tma && zp_in == 0 && C % 16 == 0 && ctx->encode_tiled != nullptr &&
        (reinterpret_cast<uintptr_t>(in) & 15u) == 0 && H < (1 << 20) && W < (1 << 20)) {
      DwTmaTile t;
      // channel chunk: as many channel groups per CTA as fit 256 threads next to a column tile
      // that wastes the fewest threads (a tile is strips of 4 output columns)
      int best_cb = 0;
      double best_waste = 0.0;
      for (int cb = 16; cb <= 256 && cb <= C; cb <<= 1) {  // (a TMA box holds at most 256 elements per dimension)
        if (C % cb != 0) continue;
        const int strips = DW_THREADS / (cb / 4);
        if (strips < 1) continue;
        int owt = strips * 4;
        if (stride_h == 2 && owt * 2 + 1 > 256) owt = 124;  // a TMA box holds at most 256 columns
        if (stride_h == 1 && owt + 2 > 256) owt = 252;
        const int64_t tiles = ceil_div64(Wo, owt);
        const double waste = static_cast<double>(tiles * strips * 4) / static_cast<double>(Wo);
        if (best_cb == 0 || waste < best_waste - 1e-9 || (waste < best_waste + 1e-9 && cb > best_cb)) {
          best_cb = cb;
          best_waste = waste;
        }
      }
      if (best_cb != 0) {
        t.CB = best_cb;
        t.G = best_cb / 4;
        t.strips = DW_THREADS / t.G;
        t.OWT = t.strips * 4;
        if (stride_h == 2 && t.OWT * 2 + 1 > 256) { t.OWT = 124; t.strips = 31; }
        if (stride_h == 1 && t.OWT + 2 > 256) { t.OWT = 252; t.strips = 63; }
        t.TWB = stride_h == 1 ? t.OWT + 2 : t.OWT * 2 + 1;
        t.col_tiles = static_cast<int>(ceil_div64(Wo, t.OWT));
        t.chan_chunks = static_cast<int>(C / t.CB);
        const int row_bytes = t.TWB * t.CB;
        t.row_pitch = static_cast<int>(align_up(static_cast<size_t>(row_bytes), 128));
        // output rows per CTA: what ~72 KB of input rows allow (two CTAs per SM), fewer when
        // that would leave SMs without a CTA
        const int max_rows_in = std::max(3, (72 * 1024) / t.row_pitch);
        int rows_out = std::max(1, (max_rows_in - 3) / stride_h + 1);
        rows_out = static_cast<int>(std::min<int64_t>(rows_out, Ho));
        const int64_t per_seg = N * t.col_tiles * t.chan_chunks;
        while (rows_out > 2 && per_seg * ceil_div64(Ho, rows_out) < static_cast<int64_t>(ctx->dw_tma_fill) * ctx->num_sms / 4) rows_out = (rows_out + 1) / 2;
        t.rows_out = rows_out;
        t.segments = static_cast<int>(ceil_div64(Ho, rows_out));
        const int rows_in = (rows_out - 1) * stride_h + 3;
        t.ring_bytes = rows_in * t.row_pitch;
        t.status = ctx->dev_status;
        t.setup_lanes = ctx->dw_lane_setup ? 32 : 1;
        const size_t smem = static_cast<size_t>(t.ring_bytes) + sizeof(uint64_t) * rows_in + 128 /* alignment */;
        const int64_t grid64 = per_seg * t.segments;
        if (smem <= 100 * 1024 && grid64 < (1ll << 31) && row_bytes % 16 == 0) {
          CUtensorMap tmap;
          const cuuint64_t dims[4] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(W),
                                      static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(N)};
          const cuuint64_t strides[3] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(W * C),
                                         static_cast<cuuint64_t>(H * W * C)};
          const cuuint32_t box[4] = {static_cast<cuuint32_t>(t.CB), static_cast<cuuint32_t>(t.TWB), 1, 1};
          const cuuint32_t estr[4] = {1, 1, 1, 1};
          typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                            const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                            CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                            CUtensorMapFloatOOBfill);
          const CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(
              &tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<uint8_t *>(in), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
          if (r != CUDA_SUCCESS)
            return mb_fail(ctx, MB_RUNTIME_ERROR, "cuTensorMapEncodeTiled (depthwise input) failed (%d)", static_cast<int>(r));
          const int var = mb_requant_variant(right_shift, zp_out);
#define MB_DW_TMA_LAUNCH_G(S, V, GT, SLOT)                                                                   \
  do {                                                                                                      \
    auto kern = dwconv3x3_u8_tma_kernel<S, V, GT>;                                                          \
    const uint64_t bit = 1ull << (SLOT);                                                                    \
    if (!(ctx->dw_attr_mask & bit)) {                                                                       \
      MB_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 101 * 1024));    \
      ctx->dw_attr_mask |= bit;                                                                             \
    }                                                                                                       \
    MB_CUDA(ctx, mb_launch_chained(ctx, kern, dim3(static_cast<unsigned>(grid64)), dim3(DW_THREADS), smem,  \
                                   tmap, p, packed, t, weights_cached));                                    \
  } while (0)
#define MB_DW_TMA_LAUNCH(S, V) MB_DW_TMA_LAUNCH_G(S, V, 0, (S - 1) * 6 + V)
          // the packed requantization forms (what a network's layers use) with the usual group counts
          // get kernels that know the count; slots 12.. of the attribute mask
          const int gslot = t.G == 8 ? 0 : t.G == 16 ? 1 : t.G == 32 ? 2 : t.G == 64 ? 3 : -1;
          if (gslot >= 0 && (var == 4 || var == 5) && ctx->dw_fixed_groups) {
            const int slot = 12 + ((stride_h - 1) * 2 + (var - 4)) * 4 + gslot;
#define MB_DW_G4(S, V)                                                  \
  switch (gslot) {                                                      \
    case 0: MB_DW_TMA_LAUNCH_G(S, V, 8, slot); break;                   \
    case 1: MB_DW_TMA_LAUNCH_G(S, V, 16, slot); break;                  \
    case 2: MB_DW_TMA_LAUNCH_G(S, V, 32, slot); break;                  \
    default: MB_DW_TMA_LAUNCH_G(S, V, 64, slot); break;                 \
  }
            if (stride_h == 1 && var == 5) { MB_DW_G4(1, 5) }
            else if (stride_h == 1) { MB_DW_G4(1, 4) }
            else if (var == 5) { MB_DW_G4(2, 5) }
            else { MB_DW_G4(2, 4) }
#undef MB_DW_G4
          } else
          if (stride_h == 1) {
            switch (var) {
              case 5: MB_DW_TMA_LAUNCH(1, 5); break;
              case 4: MB_DW_TMA_LAUNCH(1, 4); break;
              case 3: MB_DW_TMA_LAUNCH(1, 3); break;
              case 2: MB_DW_TMA_LAUNCH(1, 2); break;
              case 1: MB_DW_TMA_LAUNCH(1, 1); break;
              default: MB_DW_TMA_LAUNCH(1, 0); break;
            }
          } else {
            switch (var) {
              case 5: MB_DW_TMA_LAUNCH(2, 5); break;
              case 4: MB_DW_TMA_LAUNCH(2, 4); break;
              case 3: MB_DW_TMA_LAUNCH(2, 3); break;
              case 2: MB_DW_TMA_LAUNCH(2, 2); break;
              case 1: MB_DW_TMA_LAUNCH(2, 1); break;
              default: MB_DW_TMA_LAUNCH(2, 0); break;
            }
          }
#undef MB_DW_TMA_LAUNCH
#undef MB_DW_TMA_LAUNCH_G
          MB_CUDA(ctx, cudaGetLastError());
          ctx->launches++;
          return MB_SUCCESS;
        }
      }
    }
    // Rows per thread: the longest runs for which all blocks are resident at once (two
    // 256-thread blocks per SM), so that there is no partial last wave; tensors too large
    // for that take runs of 16 rows.
    const int64_t per_seg = groups * ceil_div64(Wo, 4);
    const int64_t slots = static_cast<int64_t>(ctx->num_sms) * DW_BLOCKS_PER_SM * DW_THREADS * ctx->dw_waves;
    int64_t segments = slots / (per_seg * N);
    segments = std::min<int64_t>(segments, ceil_div64(Ho, 2));
    if (segments < 1) segments = ceil_div64(Ho, 16);
    const int rows = static_cast<int>(ceil_div64(Ho, segments));
    segments = ceil_div64(Ho, rows);
    const unsigned grid = static_cast<unsigned>(ceil_div64(per_seg * segments * N, DW_THREADS));
#define MB_DW_LAUNCH(S, V)                                                                   \
  MB_CUDA(ctx, mb_launch_chained(ctx, dwconv3x3_u8_kernel<S, V>, dim3(grid), dim3(DW_THREADS), 0, p, packed, rows, \
                                 static_cast<int>(segments), weights_cached))
    const int var = mb_requant_variant(right_shift, zp_out);
    if (stride_h == 1) {
      switch (var) {
        case 5: MB_DW_LAUNCH(1, 5); break;
        case 4: MB_DW_LAUNCH(1, 4); break;
        case 3: MB_DW_LAUNCH(1, 3); break;
        case 2: MB_DW_LAUNCH(1, 2); break;
        case 1: MB_DW_LAUNCH(1, 1); break;
        default: MB_DW_LAUNCH(1, 0); break;
      }
    } else {
      switch (var) {
        case 5: MB_DW_LAUNCH(2, 5); break;
        case 4: MB_DW_LAUNCH(2, 4); break;
        case 3: MB_DW_LAUNCH(2, 3); break;
        case 2: MB_DW_LAUNCH(2, 2); break;
        case 1: MB_DW_LAUNCH(2, 1); break;
        default: MB_DW_LAUNCH(2, 0); break;
      }
    }
#undef MB_DW_LAUNCH
  } else {
    const int64_t total = N * Ho * Wo * C * mult_ch;
    if (ceil_div64(total, 256) > 0x7fffffffll)
      return mb_fail(ctx, MB_UNSUPPORTED, "mb_dwconv_u8_nhwc: output too large");
    dwconv_u8_general_kernel<<<static_cast<unsigned>(ceil_div64(total, 256)), 256, 0, ctx->stream>>>(p);
  }
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  return MB_SUCCESS;
}

extern "C" {

int mb_dwconv_u8_nhwc(mb_context *ctx, const uint8_t *in, const uint8_t *filter, const int32_t *bias,
                      uint8_t *out, int64_t N, int64_t H, int64_t W, int64_t C, int64_t mult_ch,
                      int64_t KH, int64_t KW, int stride_h, int stride_w, int dil_h, int dil_w,
                      int pad_top, int pad_left, int64_t Ho, int64_t Wo, int32_t zp_in, int32_t zp_f,
                      int32_t multiplier, int32_t right_shift, int32_t zp_out,
                      int use_float_multiplier, float multiplier_f) {
  return dwconv_u8_impl(ctx, in, filter, bias, nullptr, out, N, H, W, C, mult_ch, KH, KW, stride_h,
                        stride_w, dil_h, dil_w, pad_top, pad_left, Ho, Wo, zp_in, zp_f, multiplier,
                        right_shift, zp_out, use_float_multiplier, multiplier_f);
}

int mb_dwconv_u8_nhwc_prepacked(mb_context *ctx, const uint8_t *in, const uint8_t *filter,
                                const int32_t *bias, const void *prepacked, uint8_t *out, int64_t N,
                                int64_t H, int64_t W, int64_t C, int64_t mult_ch, int64_t KH,
                                int64_t KW, int stride_h, int stride_w, int dil_h, int dil_w,
                                int pad_top, int pad_left, int64_t Ho, int64_t Wo, int32_t zp_in,
                                int32_t zp_f, int32_t multiplier, int32_t right_shift,
                                int32_t zp_out, int use_float_multiplier, float multiplier_f) {
  return dwconv_u8_impl(ctx, in, filter, bias, prepacked, out, N, H, W, C, mult_ch, KH, KW, stride_h,
                        stride_w, dil_h, dil_w, pad_top, pad_left, Ho, Wo, zp_in, zp_f, multiplier,
                        right_shift, zp_out, use_float_multiplier, multiplier_f);
}

size_t mb_dwconv3x3_u8_prepacked_bytes(int64_t C) {
  return C > 0 && C % 4 == 0 ? sizeof(uint4) * DW_PACK_ITEMS * static_cast<size_t>(C / 4) : 0;
}

int mb_dwconv3x3_u8_prepack(mb_context *ctx, const uint8_t *filter_hwim, const int32_t *bias,
                            int64_t C, int32_t zp_in, int32_t zp_f, void *prepacked) {
  if (ctx == nullptr) return MB_INVALID_ARGS;
  if (filter_hwim == nullptr || prepacked == nullptr)
    return mb_fail(ctx, MB_INVALID_ARGS, "mb_dwconv3x3_u8_prepack: null operand");
  if (C < 4 || C % 4 != 0 || C > (1 << 24) || zp_in < 0 || zp_in > 255 || zp_f < 0 || zp_f > 255 ||
      (reinterpret_cast<uintptr_t>(filter_hwim) & 3u) || (reinterpret_cast<uintptr_t>(prepacked) & 15u))
    return mb_fail(ctx, MB_UNSUPPORTED,
                   "mb_dwconv3x3_u8_prepack: needs C %% 4 == 0, zero points in 0..255, aligned pointers");
  MB_CUDA(ctx, cudaSetDevice(ctx->device));
  const int64_t groups = C / 4;
  dwconv3x3_prepack_kernel<<<static_cast<unsigned>(ceil_div64(groups, 128)), 128, 0, ctx->stream>>>(
      filter_hwim, bias, static_cast<uint4 *>(prepacked), static_cast<int>(C), zp_in, zp_f);
  MB_CUDA(ctx, cudaGetLastError());
  ctx->launches++;
  ctx->dw_prepack_mark = ctx->launches;
  return MB_SUCCESS;
}

}  // extern "C"
