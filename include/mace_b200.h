/*
 * mace_b200 — C ABI of the B200 (sm_100a) device library for MACE's
 * quantized-GEMM / convolution path.
 *
 * This is the boundary a MACE maintainer binds a "CUDA runtime" to: the C++
 * delegators and operators registered for that runtime (see
 * mace_b200/host/) call nothing but these functions.  Plain pointers and
 * sizes only; no C++ or torch types.
 *
 * Conventions
 *  - Every function returns a MaceStatus::Code integer
 *    (include/mace/public/mace.h:244-250 of the reference): 0 success,
 *    1 invalid args, 2 out of resources, 3 unsupported, 4 runtime error.
 *    Nothing throws.  mb_last_error() gives the message of the last failure.
 *  - All data pointers passed to compute functions are DEVICE pointers (from
 *    mb_malloc or any cudaMalloc'd memory of the context's device).  Work is
 *    enqueued on the context's stream; mb_stream_sync() waits for it and
 *    reports device-side failures (bounded waits that ran out).
 *  - A context is used by one host thread at a time, like one MACE engine
 *    (test/ccunit/mace/libmace/mace_api_mt_test.cc:100-110: engines may run in
 *    parallel threads, one engine is not re-entrant).  Use one context per
 *    engine / per GPU.
 *  - There is no CPU fallback: on a machine without a CUDA device mb_init
 *    fails with MB_RUNTIME_ERROR.
 */
#ifndef MACE_B200_H_
#define MACE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MB_SUCCESS = 0,
  MB_INVALID_ARGS = 1,
  MB_OUT_OF_RESOURCES = 2,
  MB_UNSUPPORTED = 3,
  MB_RUNTIME_ERROR = 4
};

typedef struct mb_context mb_context;

/* ---- runtime: replaces CpuRuntime / CpuRefAllocator ----------------------
 * (mace/runtimes/cpu/cpu_runtime.cc:28-109, cpu_ref_allocator.cc:26-40;
 * buffer mapping of a device runtime: mace/core/runtime/runtime.cc:59-82). */
int mb_init(int device, mb_context **ctx);
int mb_destroy(mb_context *ctx);
const char *mb_last_error(const mb_context *ctx);
int mb_malloc(mb_context *ctx, size_t bytes, void **dptr);
int mb_free(mb_context *ctx, void *dptr);
/* Pinned host memory for staging (Map/UnMap of a device buffer). */
int mb_host_alloc(mb_context *ctx, size_t bytes, void **hptr);
int mb_host_free(mb_context *ctx, void *hptr);
/* Asynchronous copies on the context's stream. */
int mb_memcpy_h2d(mb_context *ctx, void *dst_dev, const void *src_host, size_t bytes);
int mb_memcpy_d2h(mb_context *ctx, void *dst_host, const void *src_dev, size_t bytes);
int mb_memset(mb_context *ctx, void *dst_dev, int value, size_t bytes);
int mb_memcpy_d2d(mb_context *ctx, void *dst_dev, const void *src_dev, size_t bytes);
/* Uploads that overlap the compute stream's work (double-buffered inputs): the
 * context owns a second stream for them.
 *   mb_upload_h2d         asynchronous copy from PINNED host memory on the upload stream
 *   mb_upload_wait_event  the upload stream waits for an event recorded with mb_event_record
 *                         (i.e. on the compute stream), e.g. "the staging buffer has been
 *                         consumed", before later uploads overwrite it
 *   mb_upload_signal      the compute stream waits for every upload enqueued so far
 * None of them may be called between mb_graph_begin and mb_graph_end. */
int mb_upload_h2d(mb_context *ctx, void *dst_dev, const void *src_host, size_t bytes);
int mb_upload_wait_event(mb_context *ctx, void *event);
int mb_upload_signal(mb_context *ctx);
/* The other direction: a copy to PINNED host memory that starts when the compute stream has
 * reached this call but runs on a third stream, so the kernels enqueued behind it do not wait
 * for it; done_event (from mb_event_create, may be NULL) is recorded behind the copy.  Whoever
 * overwrites src_dev later must wait for that event: mb_stream_wait_event makes the compute
 * stream do so.  (No counterpart in the reference: its runtimes copy synchronously,
 * mace/core/runtime/runtime.h.) */
int mb_download_d2h(mb_context *ctx, void *dst_host, const void *src_dev, size_t bytes, void *done_event);
int mb_stream_wait_event(mb_context *ctx, void *event);
int mb_stream_sync(mb_context *ctx);

/* ---- Failure paths ---------------------------------------------------------
 * mb_set_runtime_failure_ratio / mb_should_mock_runtime_failure: the reference's
 * allocator fault injection (ShouldMockRuntimeFailure,
 * mace/core/runtime_failure_mock.cc:25-53, env MACE_RUNTIME_FAILURE_RATIO, checked
 * at the top of every allocator's New()).  With a ratio r in (0, 1] every mb_malloc
 * fails with MACE_OUT_OF_RESOURCES with probability r.  The ratio is process-wide;
 * it is read from the environment at the first allocation unless set here.
 *
 * mb_wait_timeout_selftest: runs the bounded mbarrier wait that the tensor-core
 * kernels use on a barrier nobody arrives at, with a budget of `budget_cycles` SM
 * clocks (1 .. 2^31), so that it runs out: the kernel records the timeout in the
 * context's status word and returns; the next mb_stream_sync then fails with
 * MACE_RUNTIME_ERROR ("a kernel gave up a bounded wait") and clears the word, and
 * the context stays usable.  No counterpart in the reference (its kernels do not
 * wait on one another); it mirrors how an error code travels up through
 * MACE_RETURN_IF_ERROR (include/mace/utils/logging.h:86-95).  host_waited_cycles
 * (may be NULL) receives the clocks the wait took. */
int mb_set_runtime_failure_ratio(float ratio);
int mb_should_mock_runtime_failure(void);
int mb_wait_timeout_selftest(mb_context *ctx, long long budget_cycles,
                             long long *host_waited_cycles);
/* The cudaStream_t of the context, as an opaque pointer (for event timing). */
void *mb_stream(mb_context *ctx);
/* Device-side timing on the context's stream (the per-operator CallStats of
 * SerialNet::Run, mace/core/net/serial_net.cc:122-180, are filled from these):
 * create two events, record one before and one after the work, then read the
 * elapsed milliseconds (waits for the second event). */
int mb_event_create(mb_context *ctx, void **event);
int mb_event_record(mb_context *ctx, void *event);
int mb_event_elapsed_ms(mb_context *ctx, void *start, void *stop, float *ms);
int mb_event_destroy(mb_context *ctx, void *event);
/* Blocks the calling host thread until the event has happened. */
int mb_event_sync(mb_context *ctx, void *event);
/* CUDA-graph capture of a sequence of calls on this context (the launch-bound
 * tail of a small-batch net costs more on the host than on the GPU).  Between
 * mb_graph_begin and mb_graph_end every call on the context is recorded
 * instead of executed; mb_graph_launch replays the recorded work.  Run the same
 * sequence once uncaptured first: a call that would have to grow the scratch
 * arena during capture fails with MB_RUNTIME_ERROR.  Pointers and shapes are
 * baked into the graph. */
int mb_graph_begin(mb_context *ctx);
int mb_graph_end(mb_context *ctx, void **graph_exec);
int mb_graph_launch(mb_context *ctx, void *graph_exec);
int mb_graph_destroy(mb_context *ctx, void *graph_exec);
/* Number of kernels launched through this context so far; the second form
 * counts only launches of the persistent tcgen05 GEMM kernels (the
 * thread-per-pixel convolution kernels, which also multiply on the tensor
 * core, are not in it). */
uint64_t mb_launch_count(const mb_context *ctx);
uint64_t mb_launch_count_tensor_core(const mb_context *ctx);
/* ... and how many of those ran on CTA pairs (see the "pair" option). */
uint64_t mb_launch_count_pair(const mb_context *ctx);
/* How many such pairs the device holds at once (0 before the first pair launch). */
int mb_pair_clusters(const mb_context *ctx);
/* Options: "tensor_cores" (1 default; 0 forces the CUDA-core GEMM, for A/B
 * tests), "mn_major" (1 default; 0 transposes MN-major operands to K-major
 * in scratch instead of describing them to the tensor core directly),
 * "col_budget_mb" (1024 default: the fp32 general convolution gathers the
 * im2col columns of as many images at a time as fit into this many MiB of
 * scratch), "wino_plane" (1 default; 0 takes the one-thread-per-tile Winograd
 * output transform instead of the plane-at-a-time one, for A/B tests), "pdl"
 * (1 default; 0 launches the kernels of the uint8 operator chain in plain
 * stream order instead of with programmatic stream serialization),
 * "dw_waves" (1 default: the 3x3 depthwise grid is sized so that all blocks
 * are resident at once; n sizes it for n such rounds with shorter row runs),
 * "pair" (0 default; 1: uint8 GEMMs of at least one round of 256 x 256 tiles
 * over the SM pairs run on clusters of two CTAs -- tcgen05.mma.cta_group::2,
 * each CTA loading half of a tile's operands; 2: wherever that kernel can
 * run, for tests.  Measured no faster than one CTA per 128 x 256 tile),
 * "split_k" (1 default: a product with fewer output tiles than a quarter of
 * the SMs and a depth of 2048 or more is computed as 4 or 8 depth runs on as
 * many times the SMs, their exact int32 results added by a second kernel;
 * 0 keeps one CTA per output tile),
 * "gemv_lhs_const" (0 default; 1 promises that the matrix of the following
 * mb_gemv_u8 calls is not written by work enqueued ahead of them -- a weight,
 * the reference's Tensor::is_weight(), mace/core/tensor.h -- so its first
 * bytes may be fetched while the previous kernel still runs; such launches use
 * 2 KB chunks so that a launch and its successor share the SMs,
 * "gemv_chain_chunks" = 0 keeps 4 KB chunks),
 * "stem_tc" (1 default: a 3x3 convolution over 3 channels whose output
 * channel count is a multiple of 16 takes one tensor-core product per 128
 * pixels; 0 keeps the dp4a kernel that serves the other channel counts),
 * "thin_pw" (1 default: a pointwise convolution of depth 32 with at most 128
 * output channels, a multiple of 16, and at least 128 pixels per SM runs on
 * the same thread-per-pixel kernel instead of the persistent GEMM, whose
 * 128-pixel tiles are mostly hand-over at that depth; 2 adds depth 64, 3
 * depth 128 -- both measured slower than the GEMM; 0 switches it off),
 * "dw_fixed_groups" (1 default: the TMA-fed 3x3 depthwise kernel takes a
 * variant that knows the number of channel groups per CTA at compile time;
 * 0 keeps the generic one, for A/B tests),
 * "dw_tma_fill" (4 default: that kernel's row runs are halved until the grid
 * has this many quarter-CTAs per SM, i.e. one CTA per SM; 8 = two per SM was
 * the earlier rule and 2.4 % slower on MobileNet-v1),
 * "dw_lane_setup" (1 default: a lane per input row requests that kernel's
 * row copies; 0: one thread does, for A/B tests),
 * "conv_filter_const" (0 default; 1 promises that filter and bias of the
 * following mb_conv2d_u8_nhwc calls are not written by work enqueued ahead
 * of them -- weights, the reference's Tensor::is_weight() -- so the
 * thread-per-pixel kernels read them before they wait for the kernel in
 * front; the Conv2d delegator sets it per call),
 * "b_prefetch" (1 default: a tensor-core GEMM whose B operand was declared
 * a weight -- conv_filter_const for 1x1 convolutions, gemv_lhs_const for a
 * batched FullyConnected -- asks for its first B tiles into L2 before it
 * waits for the kernel in front; 0 switches that off, for A/B tests),
 * "stem_grid" (1 default: the thread-per-pixel convolution kernels launch
 * this many times the blocks that are resident at once). */
int mb_set_option(mb_context *ctx, const char *name, int value);

/* ---- uint8 GEMM: replaces the gemmlowp calls of MatMulOp<RT_CPU,uint8_t>
 * (mace/ops/matmul.cc:228-309 uint8 output, :311-394 int32 output) and of
 * Conv2dOp<RT_CPU,uint8_t> (mace/ops/conv_2d.cc:301-315).
 *
 * Per batch entry: acc[m,n] = sum_k (A[m,k]-zp_a)(B[k,n]-zp_b) (+ bias),
 * C = clamp(RoundingDivideByPOT(SRDHM(acc, multiplier), right_shift) + zp_c).
 * A is M x K, row-major unless a_col_major; B is K x N; C is M x N.
 * out_is_int32: C is int32 and receives acc (+bias) unrequantized.
 * bias may be NULL; bias_per_row selects bias[m] (Conv2D's per-output-channel
 * bias on gemmlowp result rows) or bias[n].  multiplier/right_shift come from
 * GetOutputMultiplierAndShift (mace/core/quantize.h:116-126). */
int mb_gemm_u8(mb_context *ctx, const uint8_t *A, const uint8_t *B,
               const int32_t *bias, void *C, int out_is_int32, int64_t batch,
               int64_t M, int64_t N, int64_t K, int a_col_major,
               int b_col_major, int c_col_major, int a_batched, int b_batched,
               int32_t zp_a, int32_t zp_b, int32_t multiplier,
               int32_t right_shift, int32_t zp_c, int bias_per_row);

/* ---- uint8 GEMV: replaces arm::q8::Gemv / ref::q8::Gemv
 * (mace/ops/arm/q8/gemv.cc:36-171, mace/ops/ref/q8/gemv.cc:80-162), the
 * delegator behind FullyConnectedOp<RT_CPU,uint8_t>
 * (mace/ops/fully_connected.cc:141-179).
 * out[b,h] = Saturate<u8>(roundf(acc * multiplier [+ zp_out])) with the
 * product and the sum rounded separately; add_zp_out = 0 gives the REF
 * delegator's formula, which omits zp_out.  lhs is [rows x K] row-major. */
int mb_gemv_u8(mb_context *ctx, const uint8_t *lhs, const uint8_t *rhs,
               const int32_t *bias, void *out, int out_is_int32, int64_t batch,
               int64_t rows, int64_t K, int lhs_batched, int rhs_batched,
               int32_t zp_lhs, int32_t zp_rhs, float multiplier,
               int32_t zp_out, int add_zp_out);

/* ---- uint8 Conv2D, NHWC x OHWI -> NHWC: replaces Conv2dOp<RT_CPU,uint8_t>::
 * Run including its Im2col (mace/ops/conv_2d.cc:201-412).  pad_top/pad_left
 * are the leading paddings (total padding >> 1); taps outside the image
 * contribute zero, which equals padding with the input zero point. */
int mb_conv2d_u8_nhwc(mb_context *ctx, const uint8_t *in,
                      const uint8_t *filter_ohwi, const int32_t *bias,
                      uint8_t *out, int64_t N, int64_t H, int64_t W, int64_t C,
                      int64_t O, int64_t KH, int64_t KW, int stride_h,
                      int stride_w, int pad_top, int pad_left, int64_t Ho,
                      int64_t Wo, int32_t zp_in, int32_t zp_f,
                      int32_t multiplier, int32_t right_shift, int32_t zp_out);

/* ---- uint8 DepthwiseConv2d, NHWC x HWIM -> NHWC: replaces
 * DepthwiseConv2dOp<RT_CPU,uint8_t>::Run (mace/ops/depthwise_conv2d.cc:
 * 152-250, fixed-point requantization) and, with use_float_multiplier != 0,
 * its dilated fallback DepthwiseConv2dGeneral (:252-320,
 * int(round(acc * multiplier_f)) + zp_out). */
int mb_dwconv_u8_nhwc(mb_context *ctx, const uint8_t *in,
                      const uint8_t *filter_hwim, const int32_t *bias,
                      uint8_t *out, int64_t N, int64_t H, int64_t W, int64_t C,
                      int64_t channel_multiplier, int64_t KH, int64_t KW,
                      int stride_h, int stride_w, int dil_h, int dil_w,
                      int pad_top, int pad_left, int64_t Ho, int64_t Wo,
                      int32_t zp_in, int32_t zp_f, int32_t multiplier,
                      int32_t right_shift, int32_t zp_out,
                      int use_float_multiplier, float multiplier_f);

/* The 3x3 / channel-multiplier-1 / undilated / stride 1 or 2 / C % 4 == 0 case runs a
 * kernel that wants the filter (and bias) rearranged into signed 8-bit tap words per
 * channel group.  mb_dwconv_u8_nhwc prepares them on every call; a caller whose filter
 * and bias are constant (filter->is_weight(), as the CPU Winograd delegator caches its
 * transformed filter, mace/ops/arm/base/conv_2d_3x3_winograd.cc:120-145) prepares them
 * once into a buffer of mb_dwconv3x3_u8_prepacked_bytes(C) bytes (0: not eligible) and
 * passes it to mb_dwconv_u8_nhwc_prepacked; zp_in and zp_f must be the values used for
 * packing.  `prepacked` may be NULL, and is ignored when the call is not that case.
 * Precondition: the buffer must be filled by mb_dwconv3x3_u8_prepack on the SAME context
 * (or by a copy on its stream) -- the depthwise kernel reads the tap words before it has
 * waited for the kernel in front of it, unless that kernel is this context's prepack
 * kernel, which the context tracks.  A buffer written by a kernel on another stream must
 * be complete (event or sync) before the call. */
size_t mb_dwconv3x3_u8_prepacked_bytes(int64_t C);
int mb_dwconv3x3_u8_prepack(mb_context *ctx, const uint8_t *filter_hwim,
                            const int32_t *bias, int64_t C, int32_t zp_in,
                            int32_t zp_f, void *prepacked);
int mb_dwconv_u8_nhwc_prepacked(mb_context *ctx, const uint8_t *in,
                                const uint8_t *filter_hwim, const int32_t *bias,
                                const void *prepacked, uint8_t *out, int64_t N,
                                int64_t H, int64_t W, int64_t C,
                                int64_t channel_multiplier, int64_t KH, int64_t KW,
                                int stride_h, int stride_w, int dil_h, int dil_w,
                                int pad_top, int pad_left, int64_t Ho, int64_t Wo,
                                int32_t zp_in, int32_t zp_f, int32_t multiplier,
                                int32_t right_shift, int32_t zp_out,
                                int use_float_multiplier, float multiplier_f);

/* ---- uint8 average pooling, NHWC: replaces PoolingOp<RT_CPU,uint8_t> AVG
 * (mace/ops/pooling.cc:638-871): (sum + n/2) / n over the in-bounds window. */
int mb_avgpool_u8_nhwc(mb_context *ctx, const uint8_t *in, uint8_t *out,
                       int64_t N, int64_t H, int64_t W, int64_t C, int64_t KH,
                       int64_t KW, int stride_h, int stride_w, int pad_top,
                       int pad_left, int64_t Ho, int64_t Wo);

/* ---- fp32 path (NCHW activations, OIHW filters) -----------------------------
 * Activation codes are ops::ActivationType values (mace/ops/common/
 * activation_type.h:21-31): 0 NOOP, 1 RELU, 2 RELUX (max_limit), 6 LEAKYRELU
 * (coefficient).  Bias (per output channel, may be NULL) and activation are
 * fused into the producing kernel; the CPU operator runs them as two extra
 * passes (mace/ops/conv_2d.cc:171-173, ref/bias_add.cc:74-103,
 * ref/activation.cc:61-88). */

/* Batched C = A * B in fp32: replaces ref::Gemm<float> / arm::Gemm<float>
 * (mace/ops/ref/gemm.cc:57-106, mace/ops/arm/base/gemm.cc:520-683).  Any
 * row/column-major combination; A is M x K, B is K x N, C is M x N. */
int mb_gemm_f32(mb_context *ctx, const float *A, const float *B, float *C,
                int64_t batch, int64_t M, int64_t N, int64_t K, int a_col_major,
                int b_col_major, int c_col_major, int a_batched, int b_batched);

/* out[b,h] = bias[h] + sum_w lhs[h,w] * rhs[b,w]: replaces ref::Gemv<float> /
 * arm::Gemv<float> (mace/ops/ref/gemv.cc:45-81, mace/ops/arm/fp32/gemv.cc:37). */
int mb_gemv_f32(mb_context *ctx, const float *lhs, const float *rhs,
                const float *bias, float *out, int64_t batch, int64_t rows,
                int64_t K, int lhs_batched, int rhs_batched);

/* General fp32 Conv2D, NCHW x OIHW -> NCHW: replaces ref::Conv2d<float> and the
 * NEON general / 1x1 delegators (mace/ops/ref/conv_2d.cc:36-122,
 * mace/ops/arm/base/conv_2d_general.cc:26-197, conv_2d_1x1.cc:27-72).  A 1x1
 * stride-1 filter is run as a batched GEMM filter[O x C] * input_n[C x H*W]. */
int mb_conv2d_f32_nchw(mb_context *ctx, const float *in, const float *filter_oihw,
                       const float *bias, float *out, int64_t N, int64_t C,
                       int64_t H, int64_t W, int64_t O, int64_t KH, int64_t KW,
                       int stride_h, int stride_w, int dil_h, int dil_w,
                       int pad_top, int pad_left, int64_t Ho, int64_t Wo,
                       int activation, float max_limit, float coefficient);

/* The same convolution with a residual: out = act(conv(in) + bias + residual),
 * residual shaped like out.  What a net runs after merging a convolution with
 * the Eltwise SUM (and its Activation) that consumes it — a bottleneck block's
 * last 1x1 convolution and its shortcut; for 1x1 stride-1 convolutions the sum
 * and the activation run in the GEMM's epilogue, other shapes run the
 * convolution and then one sum + activation pass in place.  The values are
 * those of the separate operators: (acc + bias) + residual, then the
 * activation.  residual == NULL is mb_conv2d_f32_nchw. */
int mb_conv2d_f32_nchw_residual(mb_context *ctx, const float *in,
                                const float *filter_oihw, const float *bias,
                                const float *residual, float *out, int64_t N,
                                int64_t C, int64_t H, int64_t W, int64_t O,
                                int64_t KH, int64_t KW, int stride_h,
                                int stride_w, int dil_h, int dil_w, int pad_top,
                                int pad_left, int64_t Ho, int64_t Wo,
                                int activation, float max_limit,
                                float coefficient);

/* fp32 depthwise conv, NCHW, filter [multiplier, C, kh, kw]: replaces
 * ref::DepthwiseConv2d<float> (mace/ops/ref/depthwise_conv_2d.cc:36-125). */
int mb_dwconv_f32_nchw(mb_context *ctx, const float *in, const float *filter,
                       const float *bias, float *out, int64_t N, int64_t C,
                       int64_t H, int64_t W, int64_t channel_multiplier,
                       int64_t KH, int64_t KW, int stride_h, int stride_w,
                       int dil_h, int dil_w, int pad_top, int pad_left,
                       int64_t Ho, int64_t Wo, int activation, float max_limit,
                       float coefficient);

/* fp32 3x3 stride-1 Conv2D by Winograd, NCHW: replaces
 * arm::Conv2dK3x3Winograd<float> (mace/ops/arm/base/conv_2d_3x3_winograd.cc:
 * 31-787): F(6x6,3x3) on 8x8 input tiles when H > 16 and W > 16, else
 * F(2x2,3x3); tile_override 2 or 6 forces a size.  transformed_filter may be
 * NULL (the filter is transformed into scratch on every call) or a buffer of
 * (tile+2)^2 * O * C floats that mb_winograd_transform_filter_f32 filled, the
 * way the CPU delegator caches it for weights (:120-145). */
int mb_winograd_transform_filter_f32(mb_context *ctx, const float *filter_oihw,
                                     float *transformed, int64_t C, int64_t O,
                                     int tile);
int mb_conv3x3_winograd_f32_nchw(mb_context *ctx, const float *in,
                                 const float *filter_oihw,
                                 const float *transformed_filter,
                                 const float *bias, float *out, int64_t N,
                                 int64_t C, int64_t H, int64_t W, int64_t O,
                                 int pad_top, int pad_left, int64_t Ho,
                                 int64_t Wo, int activation, float max_limit,
                                 float coefficient, int tile_override);

/* ---- fp32 operators between the convolutions of a float network -----------
 * They keep activations on the device from the first convolution to the
 * logits. */

/* MAX / AVG pooling, NCHW: replaces PoolingOp<RT_CPU,float>::MaxPooling /
 * AvgPooling (mace/ops/pooling.cc:128-240).  pooling_type is ops::PoolingType
 * (mace/ops/common/pooling_type.h:20-23): 1 AVG, 2 MAX.  Taps outside the
 * image are skipped; AVG divides by the number of in-bounds taps. */
int mb_pooling_f32_nchw(mb_context *ctx, const float *in, float *out, int64_t N,
                        int64_t C, int64_t H, int64_t W, int64_t KH, int64_t KW,
                        int stride_h, int stride_w, int dil_h, int dil_w,
                        int pad_top, int pad_left, int64_t Ho, int64_t Wo,
                        int pooling_type);

/* Element-wise op on two tensors of the same shape, or (in1 == NULL) on a
 * tensor and scalar_input: replaces TensorEltwise / TensorScalarEltwise
 * (mace/ops/eltwise.cc:419-700).  type is ops::EltwiseType (mace/ops/common/
 * eltwise_type.h:21-38); built here: SUM 0 (has_coeff: in0 * coeff0 + in1 *
 * coeff1), SUB 1, PROD 2, DIV 3, MIN 4, MAX 5, NEG 6, ABS 7, SQR_DIFF 8,
 * CLIP 12 (coeff0 <= x <= coeff1); other types return MB_UNSUPPORTED.
 * swapped has the operator's meaning: the caller exchanged the operands, so
 * SUB and DIV compute in1 - in0 and in1 / in0 and SUM exchanges its
 * coefficients. */
int mb_eltwise_f32(mb_context *ctx, const float *in0, const float *in1,
                   float *out, int64_t size, int type, float scalar_input,
                   int has_coeff, float coeff0, float coeff1, int swapped);

/* The same followed by an activation (codes as above) in one pass: what a net
 * runs when it has merged an Eltwise with the Activation operator that
 * consumes it (a residual sum and its ReLU).  No counterpart in the CPU
 * runtime, which runs the two operators one after the other. */
int mb_eltwise_act_f32(mb_context *ctx, const float *in0, const float *in1,
                       float *out, int64_t size, int type, float scalar_input,
                       int has_coeff, float coeff0, float coeff1, int swapped,
                       int activation, float max_limit, float coefficient);

/* Standalone activation: replaces ref::Activation / arm::Activation
 * (mace/ops/ref/activation.cc:61-88) for the activation codes listed above.
 * in == out is allowed. */
int mb_activation_f32(mb_context *ctx, const float *in, float *out, int64_t size,
                      int activation, float max_limit, float coefficient);

/* Softmax over the middle dimension of [outer, classes, inner]: replaces
 * SoftmaxOp<RT_CPU,float> (mace/ops/softmax.cc:76-290): NCHW over channels is
 * (N, C, H*W); a 2-D or NHWC tensor is (rows, classes, 1).  use_log gives
 * log(softmax). */
int mb_softmax_f32(mb_context *ctx, const float *in, float *out, int64_t outer,
                   int64_t classes, int64_t inner, int use_log);

/* ---- Quantize / Dequantize: replace QuantizeUtil<float, uint8_t> as the
 * Quantize and Dequantize operators use it (mace/core/quantize.h:128-215,
 * mace/ops/quantize.cc:31-115).
 *   q = Saturate<uint8_t>(roundf(zero_point + (1 / scale) * x))
 *   x = scale * (q - zero_point)          (q uint8, or int32 with in_is_int32)
 * mb_minmax_f32 is FindMinMax (quantize.h:90-102); it waits for the stream and
 * returns the two values in HOST memory, for AdjustRange to derive scale and
 * zero point from.  It cannot be captured into a graph. */
int mb_quantize_f32_u8(mb_context *ctx, const float *in, uint8_t *out,
                       int64_t size, float scale, int32_t zero_point);
int mb_dequantize_f32(mb_context *ctx, const void *in, int in_is_int32,
                      float *out, int64_t size, float scale, int32_t zero_point);
int mb_minmax_f32(mb_context *ctx, const float *in, int64_t size,
                  float *host_min, float *host_max);
/* The bin counts SerialNet::Run logs for an operator that carries a quantize_info range
 * when MACE_LOG_TENSOR_RANGE is on (mace/core/net/serial_net.cc:200-221):
 *   bin_v = (max_v - min_v) / bins;  counts[clamp(int((x - min_v) / bin_v), 0, bins - 1)]++
 * into `bins` (<= 8192) int32 counters in HOST memory.  Waits for the stream; cannot be
 * captured into a graph. */
int mb_histogram_f32(mb_context *ctx, const float *in, int64_t size, float min_v,
                     float max_v, int bins, int32_t *host_counts);

/* ---- The pixels a strided 1x1 convolution reads, gathered once.  No operator
 * of its own in the reference: arm::Conv2dGeneral / ref::Conv2d index the input
 * with the stride (mace/ops/ref/conv_2d.cc:36-122).  A 1x1 convolution with
 * strides (sh, sw) and no padding equals a 1x1 stride-1 convolution of
 *   out[p][ho][wo] = in[p][ho * sh][wo * sw],  ho < ceil(H / sh), wo < ceil(W / sw)
 * over the N * C planes; two such convolutions of one tensor (a residual block's
 * shortcut and its first convolution) then share one gather. */
int mb_subsample_f32_nchw(mb_context *ctx, const float *in, float *out,
                          int64_t planes, int64_t H, int64_t W,
                          int stride_h, int stride_w);

/* ---- Layout conversion at the edge of a network: replaces ops::Transpose as
 * BaseFlow::TransposeInput / TransposeOutput call it for NHWC <-> NCHW
 * (mace/core/flow/base_flow.cc:131-204, mace/flows/cpu/cpu_ref_flow.cc:81-101)
 * and the Transpose operator for those permutations (mace/ops/transpose.cc).
 *   out[b][c][r] = in[b][r][c],  in [batch, rows, cols], out [batch, cols, rows]
 * NHWC -> NCHW: rows = H * W, cols = C; NCHW -> NHWC: rows = C, cols = H * W.
 * elem_bytes is 1 or 4; in and out must not overlap. */
int mb_transpose2d_batched(mb_context *ctx, const void *in, void *out,
                           int64_t batch, int64_t rows, int64_t cols,
                           int elem_bytes);

/* ---- uint8 GEMM without any allocation ------------------------------------
 * No counterpart in the reference.  For callers that may not allocate device
 * memory (a real-time loop with a fixed memory budget, a plugin inside an
 * application that owns all GPU memory, code that can run while another
 * stream is being captured): the same tensor-core GEMM and epilogue as
 * mb_gemm_u8, one batch entry, row-major C, but with its scratch (operand
 * byte sums and the kernel's status word) in a fixed array inside the
 * library instead of an mb_context arena.  It calls no cudaMalloc / cudaFree
 * and needs no mb_context; work is enqueued on `stream` (a cudaStream_t, may
 * be NULL) of the CURRENT device.
 *  - Limits: M, N <= MB_STATIC_SCRATCH_MAX_DIM; operands 16-byte aligned; K
 *    and each operand's contiguous dimension a multiple of 16; K <= 33000;
 *    zero points in 0..255.
 *    Anything else is rejected with MB_INVALID_ARGS / MB_UNSUPPORTED and a
 *    message in error_message (may be NULL).
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress); make that first call before any stream capture.
 *  - All calls on a device share the one array: calls whose kernels can
 *    overlap on the GPU (different streams or host threads) race.  Keep them
 *    on one stream or order them with events.
 *  - Every GPU that loads the library holds the array (about 130 KB) until
 *    the process exits. */
#define MB_STATIC_SCRATCH_MAX_DIM 16384
int mb_gemm_u8_static_scratch(void *stream, const uint8_t *A, const uint8_t *B,
                              const int32_t *bias, void *C, int out_is_int32,
                              int64_t M, int64_t N, int64_t K, int a_col_major,
                              int b_col_major, int32_t zp_a, int32_t zp_b,
                              int32_t multiplier, int32_t right_shift,
                              int32_t zp_c, int bias_per_row,
                              char *error_message, size_t error_message_len);

/* No counterpart in the reference.  The kernel behind mb_gemm_u8_static_scratch
 * bounds its waits; if one runs out it records a non-zero code in a status word
 * of the static array and stops early, leaving C incomplete.  That call itself
 * still returns MB_SUCCESS (the kernel runs later), so a caller that wants to
 * know asks here: the status word of the last call on the current device is
 * copied into *host_status by an asynchronous copy enqueued on `stream` (no
 * allocation).  Synchronize the stream, then read: 0 = the last GEMM ran to
 * completion; 1 / 2 / 3 = its TMA producer / MMA issuer / epilogue gave up
 * waiting.  The next mb_gemm_u8_static_scratch call clears the word. */
int mb_gemm_u8_static_scratch_status(void *stream, int *host_status);

#ifdef __cplusplus
}
#endif

#endif /* MACE_B200_H_ */
