/*
 * CPU oracle for the quantized-GEMM / convolution path of MACE.
 *
 * TEST INFRASTRUCTURE ONLY.  This library restates, in plain C++ on the host,
 * the arithmetic that MACE's CPU operators perform, so that the CUDA kernels
 * can be checked against it.  Nothing in the product library links, loads or
 * calls it; only the test-suite, the smoke check and the CPU-baseline leg of
 * the benchmark do.
 *
 * Parity pins: the quantized Conv2D known-answer test ({230},
 * test/ccunit/mace/ops/conv_2d_test.cc:1240-1275), the quantized depthwise
 * known-answer test ({255, 21}, test/ccunit/mace/ops/depthwise_conv2d_test.cc:
 * 333-372) and the fp32 literal cases of the same files.  Quantized MatMul has
 * no bit-level pin in the reference (its tests use a cosine-similarity check);
 * it shares the requantization pipeline that the Conv2D pin covers.
 *
 * Every function cites the reference file:line whose behaviour it follows.
 * All functions return 0 on success or a MaceStatus-like code
 * (1 = invalid args) and never throw.
 */
#ifndef ORACLE_ORACLE_H_
#define ORACLE_ORACLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Number of worker threads used by the threaded entry points (static range
 * split, like utils::ThreadPool::Compute1D/2D, mace/utils/thread_pool.cc:339).
 * n <= 0 selects the number of online cores.  Returns the value in effect. */
int orc_set_threads(int n);
int orc_get_threads(void);

/* ---- quantization helpers ------------------------------------------------ */

/* AdjustRange<uint8_t>, mace/core/quantize.h:29-66. */
void orc_adjust_range_u8(float in_min, float in_max, int non_zero,
                         float *scale, int32_t *zero_point);

/* Quantize with Saturate(roundf(zero_point + (1/scale) * x)),
 * mace/core/quantize.h:140-151 (QuantizeWithScaleAndZeropoint). */
void orc_quantize_u8(const float *in, int64_t n, float scale,
                     int32_t zero_point, uint8_t *out);

/* GetOutputMultiplierAndShift, mace/core/quantize.h:104-126.  Returns 1 when
 * the real multiplier is outside (0,1) (the reference aborts there). */
int orc_output_multiplier_and_shift(float lhs_scale, float rhs_scale,
                                    float out_scale, int32_t *multiplier,
                                    int32_t *right_shift);

/* The gemmlowp output stage QuantizeDownInt32ToUint8ScaleByFixedPoint followed
 * by SaturatingCastToUint8, as wired in mace/ops/common/gemmlowp_util.h:37-74:
 * clamp(RoundingDivideByPOT(SaturatingRoundingDoublingHighMul(acc, mult),
 * shift) + zp_out, 0, 255). */
uint8_t orc_requant_fixed(int32_t acc, int32_t multiplier, int32_t right_shift,
                          int32_t zp_out);

/* The same two rounding stages without the offset and the clamp:
 * RoundingDivideByPOT(SRDHM(acc, multiplier), right_shift). */
int32_t orc_rounding_stages(int32_t acc, int32_t multiplier, int32_t right_shift);

/* GetBiasData, mace/ops/arm/q8/quantization_util.cc:20-46.  bias may be NULL
 * (zeros are produced). out has `channels` entries. */
void orc_get_bias_data(const int32_t *bias, float bias_scale,
                       float input_scale, float filter_scale,
                       int64_t channels, int32_t *out);

/* CalcPaddingAndOutputSize, mace/ops/common/conv_pool_2d_util.cc:30-120.
 * padding_type: 0 VALID, 1 SAME, 2 FULL.  total padding per dimension is
 * returned; callers place pad>>1 before and the rest after. */
int orc_calc_padding_and_output_size(int64_t in_h, int64_t in_w, int64_t k_h,
                                     int64_t k_w, int dil_h, int dil_w,
                                     int stride_h, int stride_w,
                                     int padding_type, int64_t *out_h,
                                     int64_t *out_w, int *pad_h, int *pad_w);

/* ---- uint8 GEMM ---------------------------------------------------------- */

/* C = requant(sum_k (A[m,k]-zp_a)(B[k,n]-zp_b) + bias) per batch entry.
 * Follows MatMulFixpointImpl (mace/ops/matmul.cc:228-309, :311-394) and the
 * GEMM call of the quantized Conv2D (mace/ops/conv_2d.cc:301-315).
 * A is M x K (row-major unless a_col_major), B is K x N, C is M x N.
 * out_is_int32 != 0: C receives the raw int32 sums (+bias), no requantization.
 * bias may be NULL; bias_per_row != 0: bias[m], else bias[n]. */
int orc_gemm_u8(const uint8_t *A, const uint8_t *B, const int32_t *bias,
                void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N,
                int64_t K, int a_col_major, int b_col_major, int c_col_major,
                int a_batched, int b_batched, int32_t zp_a, int32_t zp_b,
                int32_t multiplier, int32_t right_shift, int32_t zp_c,
                int bias_per_row);

/* ---- uint8 GEMV ---------------------------------------------------------- */

/* arm::q8::Gemv (mace/ops/arm/q8/gemv.cc:36-171) when add_zp_out != 0,
 * ref::q8::Gemv (mace/ops/ref/q8/gemv.cc:80-162) when add_zp_out == 0:
 * out[b,h] = Saturate<uint8>(roundf(acc * multiplier_float [+ zp_out])),
 * the product and the sum each rounded to float (no fused multiply-add).
 * lhs is [rows x K] row-major (batched when lhs_batched), rhs is [K]. */
int orc_gemv_u8(const uint8_t *lhs, const uint8_t *rhs, const int32_t *bias,
                void *out, int out_is_int32, int64_t batch, int64_t rows,
                int64_t K, int lhs_batched, int rhs_batched, int32_t zp_lhs,
                int32_t zp_rhs, float multiplier, int32_t zp_out,
                int add_zp_out);

/* ---- uint8 convolutions -------------------------------------------------- */

/* Quantized Conv2D, NHWC input, OHWI filter, NHWC output; im2col with the
 * input zero point as pad value then the GEMM above
 * (mace/ops/conv_2d.cc:201-412).  pad_h/pad_w are TOTAL paddings. */
int orc_conv2d_u8_nhwc(const uint8_t *in, const uint8_t *filter,
                       const int32_t *bias, uint8_t *out, int64_t N, int64_t H,
                       int64_t W, int64_t C, int64_t O, int64_t KH, int64_t KW,
                       int stride_h, int stride_w, int pad_h, int pad_w,
                       int64_t Ho, int64_t Wo, int32_t zp_in, int32_t zp_f,
                       int32_t multiplier, int32_t right_shift,
                       int32_t zp_out);

/* Quantized depthwise conv, NHWC input, HWIM filter
 * (mace/ops/depthwise_conv2d.cc:152-250; the arithmetic of the TF-Lite
 * DepthwiseConv it calls: int32 accumulation of (in-zp_in)(f-zp_f) over the
 * in-bounds taps, + bias, fixed-point requantization, + zp_out, clamp).
 * pad_top/pad_left are the leading paddings (total >> 1). */
int orc_dwconv_u8_nhwc(const uint8_t *in, const uint8_t *filter,
                       const int32_t *bias, uint8_t *out, int64_t N, int64_t H,
                       int64_t W, int64_t C, int64_t mult_ch, int64_t KH,
                       int64_t KW, int stride_h, int stride_w, int dil_h,
                       int dil_w, int pad_top, int pad_left, int64_t Ho,
                       int64_t Wo, int32_t zp_in, int32_t zp_f,
                       int32_t multiplier, int32_t right_shift,
                       int32_t zp_out);

/* DepthwiseConv2dGeneral (mace/ops/depthwise_conv2d.cc:252-320): the dilated
 * fallback, int(round(sum * multiplier_float)) + zp_out, clamp. */
int orc_dwconv_u8_nhwc_general(const uint8_t *in, const uint8_t *filter,
                               const int32_t *bias, uint8_t *out, int64_t N,
                               int64_t H, int64_t W, int64_t C,
                               int64_t mult_ch, int64_t KH, int64_t KW,
                               int stride_h, int stride_w, int dil_h,
                               int dil_w, int pad_top, int pad_left,
                               int64_t Ho, int64_t Wo, int32_t zp_in,
                               int32_t zp_f, float multiplier,
                               int32_t zp_out);

/* Quantized global / windowed average pool, NHWC:
 * (sum + n/2) / n over the in-bounds window (mace/ops/pooling.cc:638-871). */
int orc_avgpool_u8_nhwc(const uint8_t *in, uint8_t *out, int64_t N, int64_t H,
                        int64_t W, int64_t C, int64_t KH, int64_t KW,
                        int stride_h, int stride_w, int pad_top, int pad_left,
                        int64_t Ho, int64_t Wo);

/* ---- fp32 ---------------------------------------------------------------- */

/* ref::Conv2d<float>, NCHW / OIHW, float accumulator in the order
 * c -> kh -> kw (mace/ops/ref/conv_2d.cc:36-122).  Optional bias (per output
 * channel, mace/ops/ref/bias_add.cc:74-103) and activation
 * (mace/ops/ref/activation.cc:61-88; act: 0 NOOP, 1 RELU, 2 RELUX, 6 LEAKYRELU)
 * are applied afterwards as separate passes like Conv2dOp<RT_CPU,float>::Run
 * (mace/ops/conv_2d.cc:171-173). */
int orc_conv2d_f32_nchw(const float *in, const float *filter,
                        const float *bias, float *out, int64_t N, int64_t C,
                        int64_t H, int64_t W, int64_t O, int64_t KH,
                        int64_t KW, int stride_h, int stride_w, int dil_h,
                        int dil_w, int pad_top, int pad_left, int64_t Ho,
                        int64_t Wo, int act, float max_limit, float coef);

/* ref::DepthwiseConv2d<float>, NCHW, filter [multiplier, Cin, kh, kw]
 * (mace/ops/ref/depthwise_conv_2d.cc:36-125). */
int orc_dwconv_f32_nchw(const float *in, const float *filter,
                        const float *bias, float *out, int64_t N, int64_t C,
                        int64_t H, int64_t W, int64_t mult_ch, int64_t KH,
                        int64_t KW, int stride_h, int stride_w, int dil_h,
                        int dil_w, int pad_top, int pad_left, int64_t Ho,
                        int64_t Wo, int act, float max_limit, float coef);

/* ref::Gemm<float> (mace/ops/ref/gemm.cc:57-106): float accumulator, depth
 * ascending, any row/column-major combination. */
int orc_gemm_f32(const float *A, const float *B, float *C, int64_t batch,
                 int64_t M, int64_t N, int64_t K, int a_col_major,
                 int b_col_major, int c_col_major, int a_batched,
                 int b_batched);

/* ref::Gemv<float> (mace/ops/ref/gemv.cc:45-81). */
int orc_gemv_f32(const float *lhs, const float *rhs, const float *bias,
                 float *out, int64_t batch, int64_t rows, int64_t K,
                 int lhs_batched, int rhs_batched);

/* arm::Conv2dK3x3Winograd<float> restated with scalar code
 * (mace/ops/arm/base/conv_2d_3x3_winograd.cc:31-787): 3x3, stride 1,
 * F(6,3) when the input H > 16 and W > 16, else F(2,3); U[T][O][C], V[N][T][C][tiles],
 * M[N][T][O][tiles], float accumulation.  tile_override: 0 = reference rule,
 * 2 or 6 = force that output tile size. */
int orc_conv3x3_winograd_f32_nchw(const float *in, const float *filter,
                                  const float *bias, float *out, int64_t N,
                                  int64_t C, int64_t H, int64_t W, int64_t O,
                                  int pad_top, int pad_left, int64_t Ho,
                                  int64_t Wo, int act, float max_limit,
                                  float coef, int tile_override);

/* PoolingOp<RT_CPU,float>::MaxPooling / AvgPooling (mace/ops/pooling.cc:128-240), NCHW;
 * pooling_type 1 AVG, 2 MAX (mace/ops/common/pooling_type.h:20-23). */
int orc_pooling_f32_nchw(const float *in, float *out, int64_t N, int64_t C, int64_t H, int64_t W,
                         int64_t KH, int64_t KW, int stride_h, int stride_w, int dil_h, int dil_w,
                         int pad_top, int pad_left, int64_t Ho, int64_t Wo, int pooling_type);

/* TensorEltwise / TensorScalarEltwise (mace/ops/eltwise.cc:419-700); in1 NULL = scalar form. */
int orc_eltwise_f32(const float *in0, const float *in1, float *out, int64_t size, int type,
                    float scalar_input, int has_coeff, float coeff0, float coeff1, int swapped);

/* ref::Activation (mace/ops/ref/activation.cc:61-88). */
int orc_activation_f32(const float *in, float *out, int64_t size, int act, float max_limit, float coef);

/* SoftmaxOp<RT_CPU,float> (mace/ops/softmax.cc:76-290) over the middle dimension of
 * [outer, classes, inner]. */
int orc_softmax_f32(const float *in, float *out, int64_t outer, int64_t classes, int64_t inner, int use_log);

/* QuantizeUtil::Dequantize (mace/core/quantize.h:187-197): scale * (q - zero_point). */
void orc_dequantize_u8(const uint8_t *in, int64_t n, float scale, int32_t zero_point, float *out);
void orc_dequantize_i32(const int32_t *in, int64_t n, float scale, int32_t zero_point, float *out);

#ifdef __cplusplus
}
#endif

#endif  /* ORACLE_ORACLE_H_ */
