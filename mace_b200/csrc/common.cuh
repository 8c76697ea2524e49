// Shared declarations of the device library: status codes, the context that
// every C-ABI call receives, the requantization arithmetic used by all uint8
// epilogues, and small launch helpers.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstring>
#include <string>

#include "../../include/mace_b200.h"

// Device-side status word values written by kernels whose bounded waits run
// out; the host turns any non-zero value into MB_RUNTIME_ERROR.
enum : int {
  MB_DEV_OK = 0,
  MB_DEV_TIMEOUT_PRODUCER = 1,
  MB_DEV_TIMEOUT_MMA = 2,
  MB_DEV_TIMEOUT_EPILOGUE = 3,
};

struct mb_context {
  int device = 0;
  int num_sms = 0;
  int max_smem_optin = 0;
  cudaStream_t stream = nullptr;
  cudaStream_t upload_stream = nullptr;  // created on first use: uploads that overlap the compute stream
  cudaEvent_t upload_event = nullptr;    // last mb_upload_signal
  cudaStream_t download_stream = nullptr;  // created on first use: result copies that do not hold up the compute stream
  cudaEvent_t download_event = nullptr;    // "the compute stream has reached this mb_download_d2h"
  // Scratch arena, the analogue of the runtime's RENT_SCRATCH buffers
  // (mace/core/runtime/runtime.cc:153-182): one growable device block that a
  // call carves from the start; contents do not survive the call.
  void *scratch = nullptr;
  size_t scratch_bytes = 0;
  int *dev_status = nullptr;   // device status word (bounded-wait failures)
  int *host_status = nullptr;  // pinned mirror read at sync
  void *encode_tiled = nullptr;  // cuTensorMapEncodeTiled, resolved at init
  int use_tensor_cores = 1;      // cleared by mb_set_option for A/B tests
  int use_mn_major = 1;
  uint64_t launches = 0;         // kernels launched through this context
  uint64_t launches_tc = 0;      // of which tcgen05 GEMM launches
  uint64_t launches_pair = 0;    // of which on CTA pairs (not adjusted for graph replays)
  int capturing = 0;             // inside mb_graph_begin / mb_graph_end
  long long *tc_timeline = nullptr;  // optional device buffer: per-role clock stamps of CTA 0
  uint64_t capture_launches0 = 0, capture_launches_tc0 = 0;
  uint64_t func_attr_mask = 0;   // kernels whose shared-memory limit was raised
  uint64_t func_attr_mask2 = 0;  // the same for the thread-per-pixel convolution kernels
  int pdl_next_gemm = 0;         // the next tensor-core GEMM may start before its predecessor (the
                                 // operand-sum kernel) ends; it waits for it where it reads the sums
  void *skinny_ws = nullptr;     // arrival counters of the few-row GEMM (zero between calls)
  size_t skinny_ws_bytes = 0;
  int pdl_chain = 1;             // kernels of an operator chain launched with programmatic stream
                                 // serialization (each waits for its predecessor where it first
                                 // touches global memory); 0: plain stream order
  uint64_t dw_prepack_mark = ~0ull;  // value of `launches` right after the last depthwise prepack
                                 // kernel: while they are equal that kernel is the newest one in
                                 // the stream and the depthwise kernel may not read the tap words
                                 // before it has waited for its predecessor
  int skinny_max_m = 16;         // row counts up to this take the streaming few-row GEMM
  int max_pair_clusters = 0;     // co-resident clusters of the pair GEMM (0: not asked yet)
  int stem_tc = 1;               // 3x3x3 first-layer convolution: the products on the tensor core
  int dw_tma_fill = 4;           // TMA-fed depthwise: row runs are halved until the grid has this many quarter-CTAs per SM
  int gemm_b_const = 0;          // set around a GEMM whose B operand is a weight (see conv_filter_const)
  int b_prefetch = 1;            // such a GEMM asks for its first B tiles before it waits for its predecessor (0: A/B tests)
  int conv_filter_const = 0;     // promise: filter and bias of the following mb_conv2d_u8_nhwc calls are weights
  int stem_grid = 1;             // thread-per-pixel convolution kernels: grid in multiples of the resident blocks
  int dw_lane_setup = 1;         // TMA-fed depthwise: a lane per input row requests the copies (0: one thread, for A/B)
  int dw_fixed_groups = 1;       // TMA-fed depthwise kernels specialised on the channel groups per CTA (0: generic, for A/B)
  int thin_pw = 1;               // pointwise layers of depth 32 / 64 (2: also 128) on the same thread-per-pixel kernel
  int pair_gemm = 0;             // large GEMMs on CTA pairs (clusters of two sharing each tile's B): 1 where
                                 // it applies, 2 wherever it can run.  Off by default: measured equal at 8192^3
                                 // (409 vs 410 us) and slower at 4096^3 (54.7 vs 51.6 us): the main loop is paced
                                 // by the tensor pipe at the clocks the power cap leaves, not by operand traffic
  int runs_min_m = 2;             // from this many rows on, depth runs on the tensor core replace the few-row kernel
  int split_k = 1;               // few-tile, long-depth GEMMs: cut the depth into runs over more SMs
  int gemv_stream = 1;           // one-vector GEMV through the bulk-copy streaming kernel
  int gemv_lhs_const = 0;        // the GEMV matrix is a weight: it may be fetched ahead of the dependency wait
  int gemv_chain_chunks = 1;     // constant matrix: 2 KB chunks so that a launch and its successor share the SMs
  int gemv_const_one_per_sm = 0; // with a constant matrix, leave half of each SM to the next kernel (measured slower: 6.1 vs 5.75 us per 4096 x 4096 product in a chain)
  int force_bn = 0;              // tensor-core GEMM: 64 / 128 / 256 overrides the tile-width choice
  int host_alloc_wc = 0;         // mb_host_alloc returns write-combined pinned memory
  int tc_rowsum = 1;             // short-K fused GEMM: A's row sums from 16 extra accumulator columns
  int dw_tma = 1;                // depthwise 3x3 with input zero point 0: rows through shared memory by TMA
  uint64_t dw_attr_mask = 0;     // TMA depthwise kernels whose shared-memory limit was raised
  int dw_waves = 1;              // depthwise 3x3: rounds of resident blocks the grid is sized for
  int wino_plane = 1;            // plane-at-a-time Winograd output transform (0: per-tile kernel)
  int64_t col_budget_bytes = 1ll << 30;  // im2col column matrix of the fp32 general convolution:
                                         // images are processed in chunks that stay below this
  char last_error[512] = {0};
};

int mb_fail(mb_context *ctx, int code, const char *fmt, ...);
int mb_check_cuda(mb_context *ctx, cudaError_t e, const char *what);
// Returns a device pointer to at least `bytes` of scratch (256-byte aligned),
// growing the arena if needed.  offset allows several carve-outs per call.
int mb_scratch(mb_context *ctx, size_t bytes, void **ptr);

// ---- programmatic dependent launch ------------------------------------------------------------
// A kernel launched through mb_launch_chained may be started before the kernel in front of it in
// the stream has finished: its CTAs run their prologue (barrier setup, tensor-memory
// allocation, descriptor prefetch) on SMs the predecessor has already left, and every thread
// calls mb_grid_dep_wait() before its first access to global memory, which returns when the
// predecessor has completed and its writes are visible.  mb_grid_dep_launch(), called at the top
// of a kernel, lets the kernel BEHIND it do the same.  Kernels launched the ordinary way are
// full barriers in the stream, so the two kinds mix freely.
__device__ __forceinline__ void mb_grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void mb_grid_dep_launch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
static inline cudaError_t mb_launch_chained(mb_context *ctx, void (*kern)(KArgs...), dim3 grid, dim3 block,
                                            size_t smem, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl_chain ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

#define MB_RETURN_IF_ERROR(expr)        \
  do {                                  \
    int _st = (expr);                   \
    if (_st != MB_SUCCESS) return _st;  \
  } while (0)

#define MB_CUDA(ctx, expr) MB_RETURN_IF_ERROR(mb_check_cuda((ctx), (expr), #expr))

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---- requantization arithmetic ---------------------------------------------
// gemmlowp's output stage as MACE wires it (mace/ops/common/gemmlowp_util.h:
// 37-74): SaturatingRoundingDoublingHighMul, RoundingDivideByPOT, + offset,
// clamp to [0, 255].

__device__ __forceinline__ int32_t mb_srdhm(int32_t a, int32_t b) {
  // (a*b + nudge) / 2^31 with truncating division; nudge = 2^30 when a*b >= 0,
  // 1 - 2^30 otherwise.  b is a positive multiplier in [2^30, 2^31), so the
  // a == b == INT32_MIN saturation case cannot occur.
  const int64_t ab = static_cast<int64_t>(a) * static_cast<int64_t>(b);
  const int64_t t = ab + (ab >= 0 ? (1ll << 30) : (1ll - (1ll << 30)));
  return static_cast<int32_t>(t / (1ll << 31));
}

__device__ __forceinline__ int32_t mb_rdivpot(int32_t x, int shift) {
  const int32_t mask = static_cast<int32_t>((1u << shift) - 1u);
  const int32_t remainder = x & mask;
  const int32_t threshold = (mask >> 1) + (x < 0 ? 1 : 0);
  return (x >> shift) + (remainder > threshold ? 1 : 0);
}

__device__ __forceinline__ uint32_t mb_requant(int32_t acc, int32_t mult,
                                               int shift, int32_t zp_out) {
  int32_t v = mb_rdivpot(mb_srdhm(acc, mult), shift) + zp_out;
  return static_cast<uint32_t>(min(255, max(0, v)));
}

// The same arithmetic in about a third of the instructions, for the epilogues
// that requantize hundreds of millions of values per batch.  With t = acc *
// mult (64-bit) the two rounding steps collapse into one 64-bit expression:
//   SRDHM(acc, mult)        = floor((t + 2^30) / 2^31)      (mult > 0: the
//                             truncating division with the sign-dependent
//                             nudge equals this floor for every acc)
//   RDivPOT(x, s), s >= 1   = floor((x + 2^(s-1) - [x < 0]) / 2^s)
//   floor((floor(a/m) + c) / n) = floor((a + c*m) / (m*n))
// so  y = (t + 2^30 + 2^(s+30) - [acc < 0] * 2^31) >> (31 + s)   for s >= 1
// and y = (t + 2^30) >> 31 for s == 0.  ([x < 0] and [acc < 0] differ only for
// acc = -1, mult = 2^30, where both give y = 0.)  |t| < 2^62 and the constants
// are below 2^62, so nothing overflows.  tests/test_requant_identity.py checks
// the identity against the two-step definition.
struct mb_requant_params {
  int64_t c64;   // 2^30 (+ 2^(shift+30) when shift >= 1)
  int64_t c64z;  // c64 + (zp << sh): the output zero point folded into the rounding constant
  int32_t mult;  // fixed-point multiplier in [2^30, 2^31)
  int32_t neg;   // -2^31 when shift >= 1, else 0
  int32_t sh;    // 31 + shift
  int32_t zp;    // output zero point, 0..255
};

static inline mb_requant_params mb_make_requant(int32_t mult, int32_t shift, int32_t zp_out) {
  mb_requant_params q;
  q.c64 = (1ll << 30) + (shift >= 1 ? (1ll << (shift + 30)) : 0ll);
  q.mult = mult;
  q.neg = shift >= 1 ? static_cast<int32_t>(0x80000000u) : 0;
  q.sh = 31 + shift;
  q.zp = zp_out;
  q.c64z = q.c64 + (q.sh <= 50 ? (static_cast<int64_t>(zp_out) << q.sh) : 0ll);
  return q;
}

__device__ __forceinline__ uint32_t mb_requant_fast(int32_t acc, const mb_requant_params &q) {
  int64_t t = static_cast<int64_t>(acc) * q.mult + q.c64;
  t += static_cast<int64_t>(static_cast<int32_t>(static_cast<uint32_t>(acc) >> 31)) * q.neg;
  const int32_t y = static_cast<int32_t>(t >> q.sh);
  // clamp(y + zp, 0, 255); y is capped first so that y + zp cannot wrap
  return static_cast<uint32_t>(__viaddmin_s32_relu(min(y, 255), q.zp, 255));
}

// Compile-time variants of the same expression.  SGE1 (shift >= 1): the total shift is at
// least 32, so y is the high word of t shifted by (shift - 1) -- one multiply-add and one
// 32-bit shift.  ZP0 (output zero point 0): a negative accumulator gives y <= 0 with or
// without the [acc < 0] term and clamps to 0, so the term is dropped.
template <bool ZP0, bool SGE1>
__device__ __forceinline__ uint32_t mb_requant_t(int32_t acc, const mb_requant_params &q) {
  int64_t t = static_cast<int64_t>(acc) * q.mult + q.c64;
  if (!ZP0 && SGE1)
    t += static_cast<int64_t>(static_cast<int32_t>(static_cast<uint32_t>(acc) >> 31)) * q.neg;
  const int32_t y = SGE1 ? (static_cast<int32_t>(t >> 32) >> (q.sh - 32)) : static_cast<int32_t>(t >> 31);
  if (ZP0) return static_cast<uint32_t>(__vimin_s32_relu(y, 255));
  return static_cast<uint32_t>(__viaddmin_s32_relu(min(y, 255), q.zp, 255));
}

// Four values at once for 1 <= shift <= 19: the zero point rides in the rounding constant
// (c64z), so y + zp comes straight out of the shift, and cvt.pack saturates two values to
// [0, 255] AND packs them in one instruction: 2.5 instructions per value instead of 3.75.
// (shift 0 is excluded because y + zp could wrap int32 there; shift > 19 because zp << sh
// would not fit.)
__device__ __forceinline__ uint32_t mb_pack4_sat_u8(int32_t v0, int32_t v1, int32_t v2, int32_t v3) {
  uint32_t hi, d;
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(v3), "r"(v2), "r"(0));
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(v1), "r"(v0), "r"(hi));
  return d;
}

template <bool ZP0>
__device__ __forceinline__ int32_t mb_requant_unclamped(int32_t acc, const mb_requant_params &q) {
  int64_t t = static_cast<int64_t>(acc) * q.mult + q.c64z;
  if (!ZP0) t += static_cast<int64_t>(static_cast<int32_t>(static_cast<uint32_t>(acc) >> 31)) * q.neg;
  return static_cast<int32_t>(t >> 32) >> (q.sh - 32);
}

template <bool ZP0>
__device__ __forceinline__ uint32_t mb_requant_pack4(int32_t a0, int32_t a1, int32_t a2, int32_t a3,
                                                     const mb_requant_params &q) {
  return mb_pack4_sat_u8(mb_requant_unclamped<ZP0>(a0, q), mb_requant_unclamped<ZP0>(a1, q),
                         mb_requant_unclamped<ZP0>(a2, q), mb_requant_unclamped<ZP0>(a3, q));
}

// Variant index for kernels that switch on it once per tile or thread:
//   0..3: bit 0 = ZP0, bit 1 = SGE1 (mb_requant_t);  4 / 5: packed form, zero point != 0 / == 0.
static inline int mb_requant_variant(int32_t shift, int32_t zp_out) {
  if (shift >= 1 && shift <= 19) return zp_out == 0 ? 5 : 4;
  return (zp_out == 0 ? 1 : 0) | (shift >= 1 ? 2 : 0);
}

// Saturate<uint8_t>(roundf(v)) of mace/core/quantize.h:69-83.
__device__ __forceinline__ uint32_t mb_saturate_round_u8(float v) {
  const int r = static_cast<int>(roundf(v));
  return static_cast<uint32_t>(min(255, max(0, r)));
}

// ---- fp32 epilogue ----------------------------------------------------------
// ref::Activation (mace/ops/ref/activation.cc:61-88) for the types the fp32 kernels fuse:
// 0 NOOP, 1 RELU, 2 RELUX (max_limit), 6 LEAKYRELU (coef).
__device__ __forceinline__ float mb_activate(float x, int act, float max_limit, float coef) {
  switch (act) {
    case 1: return fmaxf(0.f, x);
    case 2: return fmaxf(0.f, fminf(max_limit, x));
    case 6: return fmaxf(x, 0.f) + fminf(x, 0.f) * coef;
    default: return x;
  }
}
