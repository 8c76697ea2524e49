// Host-side scalar helpers of the quantized path: the derivation of the
// fixed-point output multiplier, padding/output-size arithmetic and the major
// order / padding enums.  Same names and argument meaning as
//   mace/core/quantize.h:104-126          (QuantizeMultiplier, GetOutputMultiplierAndShift)
//   mace/ops/common/conv_pool_2d_util.h:27-37, .cc:30-221 (Padding, RoundType,
//                                          CalcPaddingAndOutputSize, CalcOutputSize)
//   mace/ops/common/matrix.h:22-30        (MatrixMajor)
#ifndef MACE_B200_HOST_QUANTIZE_UTIL_H_
#define MACE_B200_HOST_QUANTIZE_UTIL_H_

#include <algorithm>
#include <cmath>

#include "core.h"

namespace mace {

enum Padding { VALID = 0, SAME = 1, FULL = 2 };
enum RoundType { FLOOR = 0, CEIL = 1 };
enum PoolingType { AVG = 1, MAX = 2 };

namespace ops {
enum MatrixMajor { RowMajor, ColMajor };
}  // namespace ops

// multiplier in [0.5, 1) * 2^31 and a binary exponent, from a double.
// AdjustRange<uint8_t> (mace/core/quantize.h:28-66): the range is widened to contain 0, which
// must quantize to an integer; non_zero nudges the minimum so that it quantizes to >= 1.
inline void AdjustRangeU8(const float in_min_data, const float in_max_data, const bool non_zero,
                          float *scale, int32_t *zero_point) {
  const int quantized_min = 0, quantized_max = 255;
  float out_max = std::max(0.f, in_max_data);
  float out_min = std::min(0.f, in_min_data);
  if (non_zero)
    out_min = std::min(out_min, in_min_data - (out_max - in_min_data) / (quantized_max - quantized_min - 1));
  *scale = (out_max - out_min) / (quantized_max - quantized_min);
  const float kEps = 1e-6;
  if (out_min < -kEps && out_max > kEps) {
    const float quantized_zero = -out_min / *scale;
    const int32_t near_int = static_cast<int32_t>(roundf(quantized_zero));
    *zero_point = near_int;
    if (fabs(quantized_zero - near_int) > kEps && non_zero) *zero_point = static_cast<int32_t>(std::ceil(quantized_zero));
  } else if (out_min > -kEps) {
    *zero_point = quantized_min;
  } else {
    *zero_point = quantized_max;
  }
}

inline void QuantizeMultiplier(double multiplier, int32_t *output_multiplier, int32_t *shift) {
  int exponent = 0;
  const double mantissa = std::frexp(multiplier, &exponent);
  int64_t fixed = static_cast<int64_t>(roundl(mantissa * static_cast<double>(1ll << 31)));
  if (fixed == (1ll << 31)) {  // mantissa rounded up to 1.0
    fixed /= 2;
    ++exponent;
  }
  *output_multiplier = static_cast<int32_t>(fixed);
  *shift = exponent;
}

// The real multiplier is formed in float32, as the reference does, before it is
// widened to double; it must lie in (0, 1).
inline MaceStatus GetOutputMultiplierAndShift(const float lhs_scale, const float rhs_scale,
                                              const float output_scale,
                                              int32_t *quantized_multiplier, int *right_shift) {
  const float real_multiplier = lhs_scale * rhs_scale / output_scale;
  if (!(real_multiplier > 0.f && real_multiplier < 1.f)) {
    return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "output multiplier outside (0, 1)");
  }
  int32_t exponent = 0;
  QuantizeMultiplier(real_multiplier, quantized_multiplier, &exponent);
  *right_shift = -exponent;
  if (*right_shift < 0) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "negative right shift");
  return MaceStatus::MACE_SUCCESS;
}

namespace ops {

// Output height/width and TOTAL padding for VALID / SAME / FULL; callers put
// padding >> 1 in front and the remainder behind.  height/width of the
// input and of the (dilated) kernel are passed directly.
inline MaceStatus CalcPaddingAndOutputSize(index_t in_h, index_t in_w, index_t k_h, index_t k_w,
                                           const int *dilations, const int *strides,
                                           Padding padding, index_t *out_h, index_t *out_w,
                                           int *padding_size) {
  if (dilations[0] <= 0 || dilations[1] <= 0 || strides[0] <= 0 || strides[1] <= 0 ||
      !((dilations[0] == 1 || strides[0] == 1) && (dilations[1] == 1 || strides[1] == 1))) {
    return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "invalid strides / dilations");
  }
  const index_t ext_h = (k_h - 1) * dilations[0] + 1, ext_w = (k_w - 1) * dilations[1] + 1;
  switch (padding) {
    case VALID:
      *out_h = (in_h - ext_h) / strides[0] + 1;
      *out_w = (in_w - ext_w) / strides[1] + 1;
      break;
    case SAME:
      *out_h = (in_h - 1) / strides[0] + 1;
      *out_w = (in_w - 1) / strides[1] + 1;
      break;
    case FULL:
      *out_h = (in_h + ext_h - 2) / strides[0] + 1;
      *out_w = (in_w + ext_w - 2) / strides[1] + 1;
      break;
    default:
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "unsupported padding type");
  }
  padding_size[0] = static_cast<int>(std::max<index_t>(0, (*out_h - 1) * strides[0] + ext_h - in_h));
  padding_size[1] = static_cast<int>(std::max<index_t>(0, (*out_w - 1) * strides[1] + ext_w - in_w));
  return MaceStatus::MACE_SUCCESS;
}

// Output size for explicit total paddings ("padding_values").
inline void CalcOutputSize(index_t in_h, index_t in_w, index_t k_h, index_t k_w,
                           const int *padding_size, const int *dilations, const int *strides,
                           RoundType round_type, index_t *out_h, index_t *out_w) {
  const double h = 1.0 * (in_h + padding_size[0] - k_h - (k_h - 1) * (dilations[0] - 1)) / strides[0];
  const double w = 1.0 * (in_w + padding_size[1] - k_w - (k_w - 1) * (dilations[1] - 1)) / strides[1];
  if (round_type == FLOOR) {
    *out_h = static_cast<index_t>(std::floor(h) + 1);
    *out_w = static_cast<index_t>(std::floor(w) + 1);
  } else {
    *out_h = static_cast<index_t>(std::ceil(h) + 1);
    *out_w = static_cast<index_t>(std::ceil(w) + 1);
  }
}

}  // namespace ops
}  // namespace mace

#endif  // MACE_B200_HOST_QUANTIZE_UTIL_H_
