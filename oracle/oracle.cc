// CPU oracle for the quantized-GEMM / convolution path of MACE.
//
// TEST INFRASTRUCTURE ONLY: a host restatement of the arithmetic of MACE's CPU
// operators, used as the checker for the CUDA kernels and as the timed CPU
// baseline.  The product library never links or loads it.  See oracle.h for
// the list of known-answer tests that pin it.
//
// Build with -ffp-contract=off: several reference formulas (GEMV
// requantization, Winograd transforms) are written as separate multiply and add
// operations, and the oracle keeps each rounding step.

#include "oracle.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <limits>
#include <thread>
#include <vector>

namespace {

int g_threads = 0;

int effective_threads() {
  if (g_threads > 0) return g_threads;
  unsigned n = std::thread::hardware_concurrency();
  return n == 0 ? 1 : static_cast<int>(n);
}

// Static range split over [0, n): the same partitioning idea as
// utils::ThreadPool::Compute1D (mace/utils/thread_pool.cc:339).
void parallel_for(int64_t n, const std::function<void(int64_t, int64_t)> &fn) {
  int t = effective_threads();
  if (t <= 1 || n <= 1) {
    fn(0, n);
    return;
  }
  if (t > n) t = static_cast<int>(n);
  std::vector<std::thread> pool;
  pool.reserve(t);
  const int64_t chunk = (n + t - 1) / t;
  for (int i = 0; i < t; ++i) {
    const int64_t b = i * chunk;
    const int64_t e = std::min<int64_t>(n, b + chunk);
    if (b >= e) break;
    pool.emplace_back([=, &fn]() { fn(b, e); });
  }
  for (auto &th : pool) th.join();
}

// Saturate<uint8_t>, mace/core/quantize.h:69-78: truncating cast to int, then
// clamp.
inline uint8_t saturate_u8(float value) {
  int r = static_cast<int>(value);
  if (r <= 0) return 0;
  if (r >= 255) return 255;
  return static_cast<uint8_t>(r);
}

// gemmlowp fixed-point primitive SaturatingRoundingDoublingHighMul: a*b / 2^31
// rounded to nearest, evaluated in 64 bits as (a*b + nudge) / 2^31 with a
// truncating division, nudge = 2^30 for a*b >= 0 and 1 - 2^30 otherwise (so
// exact ties round towards +infinity: 0.5 -> 1, -0.5 -> 0); saturates only for
// a == b == INT32_MIN.
inline int32_t srdhm(int32_t a, int32_t b) {
  const bool overflow = (a == b) && (a == std::numeric_limits<int32_t>::min());
  const int64_t ab = static_cast<int64_t>(a) * static_cast<int64_t>(b);
  const int32_t nudge = ab >= 0 ? (1 << 30) : (1 - (1 << 30));
  const int32_t r = static_cast<int32_t>((ab + nudge) / (1ll << 31));
  return overflow ? std::numeric_limits<int32_t>::max() : r;
}

// gemmlowp fixed-point primitive RoundingDivideByPOT: x / 2^exponent, rounding
// to nearest with ties away from zero.
inline int32_t rdivpot(int32_t x, int exponent) {
  const int32_t mask = static_cast<int32_t>((1ll << exponent) - 1);
  const int32_t remainder = x & mask;
  const int32_t threshold = (mask >> 1) + (x < 0 ? 1 : 0);
  return (x >> exponent) + (remainder > threshold ? 1 : 0);
}

inline uint8_t requant_fixed(int32_t acc, int32_t mult, int32_t shift,
                             int32_t zp_out) {
  int32_t v = rdivpot(srdhm(acc, mult), shift) + zp_out;
  return static_cast<uint8_t>(std::min(255, std::max(0, v)));
}

inline float activate(float x, int act, float max_limit, float coef) {
  // mace/ops/ref/activation.cc:61-88 (ActivationType values from
  // mace/ops/common/activation_type.h: NOOP 0, RELU 1, RELUX 2, LEAKYRELU 6).
  switch (act) {
    case 1: return std::max(0.f, x);
    case 2: return std::max(0.f, std::min(max_limit, x));
    case 6: return std::max(x, 0.f) + std::min(x, 0.f) * coef;
    default: return x;
  }
}

void bias_act_nchw(float *out, const float *bias, int64_t N, int64_t O,
                   int64_t image, int act, float max_limit, float coef) {
  if (bias == nullptr && act == 0) return;
  parallel_for(N * O, [&](int64_t b, int64_t e) {
    for (int64_t i = b; i < e; ++i) {
      const float bv = bias ? bias[i % O] : 0.f;
      float *p = out + i * image;
      for (int64_t j = 0; j < image; ++j) {
        float v = p[j];
        if (bias) v = v + bv;
        p[j] = activate(v, act, max_limit, coef);
      }
    }
  });
}

// Exact dot product of two uint8 rows in 32-bit unsigned arithmetic (the
// compiler vectorizes this to 16-bit multiply-add pairs).
inline uint32_t dot_u8(const uint8_t *a, const uint8_t *b, int64_t k) {
  uint32_t s = 0;
  for (int64_t i = 0; i < k; ++i) {
    s += static_cast<uint32_t>(static_cast<uint16_t>(a[i]) *
                               static_cast<uint16_t>(b[i]));
  }
  return s;
}

inline uint32_t sum_u8(const uint8_t *a, int64_t k) {
  uint32_t s = 0;
  for (int64_t i = 0; i < k; ++i) s += a[i];
  return s;
}

// Copy an M x K matrix into K-major (row-major M x K) storage.
void to_k_major_rows(const uint8_t *src, bool col_major, int64_t rows,
                     int64_t k, std::vector<uint8_t> *dst) {
  dst->resize(static_cast<size_t>(rows) * k);
  if (!col_major) {
    std::memcpy(dst->data(), src, static_cast<size_t>(rows) * k);
    return;
  }
  // col-major rows x k: element (r, d) at src[d * rows + r]
  uint8_t *d = dst->data();
  parallel_for(rows, [&](int64_t b, int64_t e) {
    for (int64_t r = b; r < e; ++r)
      for (int64_t kk = 0; kk < k; ++kk) d[r * k + kk] = src[kk * rows + r];
  });
}

// Core exact GEMM on K-major operands.  a: M x K rows, bt: N x K rows.
// acc(m, n) = sum_k (a - zp_a)(b - zp_b) computed as
// dot - zp_b * rowsum(a) - zp_a * rowsum(bt) + K * zp_a * zp_b; every term is
// exact in 32-bit two's-complement arithmetic whenever the true sum fits.
template <typename Emit>
void gemm_kmajor(const uint8_t *a, const uint8_t *bt, int64_t M, int64_t N,
                 int64_t K, int32_t zp_a, int32_t zp_b, Emit emit) {
  std::vector<uint32_t> sum_a(M), sum_b(N);
  for (int64_t m = 0; m < M; ++m) sum_a[m] = sum_u8(a + m * K, K);
  for (int64_t n = 0; n < N; ++n) sum_b[n] = sum_u8(bt + n * K, K);
  const uint32_t kzz = static_cast<uint32_t>(K) * static_cast<uint32_t>(zp_a) *
                       static_cast<uint32_t>(zp_b);
  const int64_t MB = 32, NB = 64;
  const int64_t mblocks = (M + MB - 1) / MB;
  const int64_t nblocks = (N + NB - 1) / NB;
  parallel_for(mblocks * nblocks, [&](int64_t b, int64_t e) {
    for (int64_t blk = b; blk < e; ++blk) {
      const int64_t m0 = (blk / nblocks) * MB, n0 = (blk % nblocks) * NB;
      const int64_t m1 = std::min(M, m0 + MB), n1 = std::min(N, n0 + NB);
      for (int64_t m = m0; m < m1; ++m) {
        for (int64_t n = n0; n < n1; ++n) {
          uint32_t d = dot_u8(a + m * K, bt + n * K, K);
          uint32_t acc = d - static_cast<uint32_t>(zp_b) * sum_a[m] -
                         static_cast<uint32_t>(zp_a) * sum_b[n] + kzz;
          emit(m, n, static_cast<int32_t>(acc));
        }
      }
    }
  });
}

}  // namespace

extern "C" {

int orc_set_threads(int n) {
  g_threads = n;
  return effective_threads();
}

int orc_get_threads(void) { return effective_threads(); }

void orc_adjust_range_u8(float in_min_data, float in_max_data, int non_zero,
                         float *scale, int32_t *zero_point) {
  const uint8_t quantized_min = 0;
  const uint8_t quantized_max = 255;
  float out_max = std::max(0.f, in_max_data);
  float out_min = std::min(0.f, in_min_data);
  if (non_zero) {
    out_min = std::min(out_min,
                       in_min_data - (out_max - in_min_data) /
                                         (quantized_max - quantized_min - 1));
  }
  *scale = (out_max - out_min) / (quantized_max - quantized_min);
  const float kEps = 1e-6;
  if (out_min < -kEps && out_max > kEps) {
    float quantized_zero = -out_min / *scale;
    int32_t near_int = static_cast<int32_t>(roundf(quantized_zero));
    *zero_point = near_int;
    if (fabs(quantized_zero - near_int) > kEps && non_zero) {
      *zero_point = static_cast<int32_t>(std::ceil(quantized_zero));
    }
  } else if (out_min > -kEps) {
    *zero_point = quantized_min;
  } else {
    *zero_point = quantized_max;
  }
}

void orc_quantize_u8(const float *in, int64_t n, float scale,
                     int32_t zero_point, uint8_t *out) {
  float recip_scale = 1 / scale;
  for (int64_t i = 0; i < n; ++i)
    out[i] = saturate_u8(roundf(zero_point + recip_scale * in[i]));
}

int orc_output_multiplier_and_shift(float lhs_scale, float rhs_scale,
                                    float out_scale, int32_t *multiplier,
                                    int32_t *right_shift) {
  float real_multiplier = lhs_scale * rhs_scale / out_scale;
  if (!(real_multiplier > 0.f && real_multiplier < 1.f)) return 1;
  int exponent;
  const double q = std::frexp(static_cast<double>(real_multiplier), &exponent);
  int64_t qint = static_cast<int64_t>(roundl(q * (1ll << 31)));
  if (qint == (1ll << 31)) {
    qint /= 2;
    ++exponent;
  }
  *multiplier = static_cast<int32_t>(qint);
  *right_shift = -exponent;
  return *right_shift >= 0 ? 0 : 1;
}

uint8_t orc_requant_fixed(int32_t acc, int32_t multiplier, int32_t right_shift,
                          int32_t zp_out) {
  return requant_fixed(acc, multiplier, right_shift, zp_out);
}

int32_t orc_rounding_stages(int32_t acc, int32_t multiplier, int32_t right_shift) {
  return rdivpot(srdhm(acc, multiplier), right_shift);
}

void orc_get_bias_data(const int32_t *bias, float bias_scale, float input_scale,
                       float filter_scale, int64_t channels, int32_t *out) {
  if (bias == nullptr) {
    std::fill_n(out, channels, 0);
    return;
  }
  bool adjust = fabs(input_scale * filter_scale - bias_scale) > 1e-6;
  if (!adjust) {
    std::copy_n(bias, channels, out);
    return;
  }
  float adjust_scale = bias_scale / (input_scale * filter_scale);
  for (int64_t i = 0; i < channels; ++i)
    out[i] = static_cast<int32_t>(roundf(bias[i] * adjust_scale));
}

int orc_calc_padding_and_output_size(int64_t in_h, int64_t in_w, int64_t k_h,
                                     int64_t k_w, int dil_h, int dil_w,
                                     int stride_h, int stride_w,
                                     int padding_type, int64_t *out_h,
                                     int64_t *out_w, int *pad_h, int *pad_w) {
  if (dil_h <= 0 || dil_w <= 0 || stride_h <= 0 || stride_w <= 0) return 1;
  if (!((dil_h == 1 || stride_h == 1) && (dil_w == 1 || stride_w == 1)))
    return 1;
  const int64_t keh = (k_h - 1) * dil_h + 1;
  const int64_t kew = (k_w - 1) * dil_w + 1;
  int64_t oh, ow;
  switch (padding_type) {
    case 0:
      oh = (in_h - keh) / stride_h + 1;
      ow = (in_w - kew) / stride_w + 1;
      break;
    case 1:
      oh = (in_h - 1) / stride_h + 1;
      ow = (in_w - 1) / stride_w + 1;
      break;
    case 2:
      oh = (in_h + keh - 2) / stride_h + 1;
      ow = (in_w + kew - 2) / stride_w + 1;
      break;
    default:
      return 1;
  }
  *pad_h = static_cast<int>(
      std::max<int64_t>(0, (oh - 1) * stride_h + keh - in_h));
  *pad_w = static_cast<int>(
      std::max<int64_t>(0, (ow - 1) * stride_w + kew - in_w));
  *out_h = oh;
  *out_w = ow;
  return 0;
}

int orc_gemm_u8(const uint8_t *A, const uint8_t *B, const int32_t *bias,
                void *C, int out_is_int32, int64_t batch, int64_t M, int64_t N,
                int64_t K, int a_col_major, int b_col_major, int c_col_major,
                int a_batched, int b_batched, int32_t zp_a, int32_t zp_b,
                int32_t multiplier, int32_t right_shift, int32_t zp_c,
                int bias_per_row) {
  if (batch < 0 || M < 0 || N < 0 || K < 0) return 1;
  std::vector<uint8_t> a_pack, bt_pack;
  for (int64_t b = 0; b < batch; ++b) {
    const uint8_t *a = A + (a_batched ? b * M * K : 0);
    const uint8_t *bm = B + (b_batched ? b * K * N : 0);
    if (b == 0 || a_batched) to_k_major_rows(a, a_col_major != 0, M, K, &a_pack);
    // B is K x N; its transpose N x K is "col-major K x N" read as rows.
    // row-major K x N == col-major N x K, so the flags invert.
    if (b == 0 || b_batched)
      to_k_major_rows(bm, b_col_major == 0, N, K, &bt_pack);
    uint8_t *c8 = static_cast<uint8_t *>(C) + b * M * N;
    int32_t *c32 = static_cast<int32_t *>(C) + b * M * N;
    gemm_kmajor(a_pack.data(), bt_pack.data(), M, N, K, zp_a, zp_b,
                [&](int64_t m, int64_t n, int32_t acc) {
                  if (bias) acc += bias_per_row ? bias[m] : bias[n];
                  const int64_t idx = c_col_major ? n * M + m : m * N + n;
                  if (out_is_int32)
                    c32[idx] = acc;
                  else
                    c8[idx] = requant_fixed(acc, multiplier, right_shift, zp_c);
                });
  }
  return 0;
}

int orc_gemv_u8(const uint8_t *lhs, const uint8_t *rhs, const int32_t *bias,
                void *out, int out_is_int32, int64_t batch, int64_t rows,
                int64_t K, int lhs_batched, int rhs_batched, int32_t zp_lhs,
                int32_t zp_rhs, float multiplier, int32_t zp_out,
                int add_zp_out) {
  if (batch < 0 || rows < 0 || K < 0) return 1;
  for (int64_t b = 0; b < batch; ++b) {
    const uint8_t *rb = rhs + (rhs_batched ? b * K : 0);
    const uint32_t sum_rhs = sum_u8(rb, K);
    parallel_for(rows, [&](int64_t hb, int64_t he) {
      for (int64_t h = hb; h < he; ++h) {
        const uint8_t *lp = lhs + (lhs_batched ? b * rows * K : 0) + h * K;
        uint32_t dot = dot_u8(lp, rb, K);
        uint32_t sum_lhs = sum_u8(lp, K);
        const int32_t zero_point_dot =
            static_cast<int32_t>(zp_lhs * zp_rhs * K);
        int32_t ret = static_cast<int32_t>(
            dot - sum_lhs * static_cast<uint32_t>(zp_rhs) -
            sum_rhs * static_cast<uint32_t>(zp_lhs) +
            static_cast<uint32_t>(zero_point_dot));
        if (bias) ret += bias[h];
        if (out_is_int32) {
          static_cast<int32_t *>(out)[b * rows + h] = ret;
        } else {
          float v = ret * multiplier;
          if (add_zp_out) v = v + zp_out;
          static_cast<uint8_t *>(out)[b * rows + h] =
              saturate_u8(std::roundf(v));
        }
      }
    });
  }
  return 0;
}

int orc_conv2d_u8_nhwc(const uint8_t *in, const uint8_t *filter,
                       const int32_t *bias, uint8_t *out, int64_t N, int64_t H,
                       int64_t W, int64_t C, int64_t O, int64_t KH, int64_t KW,
                       int stride_h, int stride_w, int pad_h, int pad_w,
                       int64_t Ho, int64_t Wo, int32_t zp_in, int32_t zp_f,
                       int32_t multiplier, int32_t right_shift,
                       int32_t zp_out) {
  const int64_t depth = C * KH * KW;
  const int64_t columns = N * Ho * Wo;
  const bool im2col_required = KH != 1 || KW != 1 || stride_h != 1 ||
                               stride_w != 1;
  const uint8_t *gemm_in = in;
  std::vector<uint8_t> col;
  if (im2col_required) {
    col.resize(static_cast<size_t>(depth) * columns);
    const uint8_t padv = static_cast<uint8_t>(zp_in);
    uint8_t *cd = col.data();
    parallel_for(N * Ho, [&](int64_t rb, int64_t re) {
      for (int64_t r = rb; r < re; ++r) {
        const int64_t b = r / Ho, h = r % Ho;
        for (int64_t w = 0; w < Wo; ++w) {
          uint8_t *dst = cd + ((b * Ho + h) * Wo + w) * depth;
          const int64_t ih0 = h * stride_h - (pad_h >> 1);
          const int64_t iw0 = w * stride_w - (pad_w >> 1);
          for (int64_t kh = 0; kh < KH; ++kh) {
            for (int64_t kw = 0; kw < KW; ++kw) {
              const int64_t ih = ih0 + kh, iw = iw0 + kw;
              uint8_t *d = dst + (kh * KW + kw) * C;
              if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
                std::memcpy(d, in + ((b * H + ih) * W + iw) * C, C);
              } else {
                std::memset(d, padv, C);
              }
            }
          }
        }
      }
    });
    gemm_in = cd;
  } else {
    if (Ho != H || Wo != W) return 1;
  }
  // filter: row-major [O x depth] (lhs); input: col-major [depth x columns]
  // (rhs); output: col-major [O x columns]; bias per result row
  // (mace/ops/conv_2d.cc:301-315).
  return orc_gemm_u8(filter, gemm_in, bias, out, 0, 1, O, columns, depth, 0, 1,
                     1, 0, 0, zp_f, zp_in, multiplier, right_shift, zp_out, 1);
}

int orc_dwconv_u8_nhwc(const uint8_t *in, const uint8_t *filter,
                       const int32_t *bias, uint8_t *out, int64_t N, int64_t H,
                       int64_t W, int64_t C, int64_t mult_ch, int64_t KH,
                       int64_t KW, int stride_h, int stride_w, int dil_h,
                       int dil_w, int pad_top, int pad_left, int64_t Ho,
                       int64_t Wo, int32_t zp_in, int32_t zp_f,
                       int32_t multiplier, int32_t right_shift,
                       int32_t zp_out) {
  const int64_t OC = C * mult_ch;
  parallel_for(N * Ho, [&](int64_t rb, int64_t re) {
    std::vector<int32_t> acc(OC);
    for (int64_t r = rb; r < re; ++r) {
      const int64_t b = r / Ho, h = r % Ho;
      for (int64_t w = 0; w < Wo; ++w) {
        std::fill(acc.begin(), acc.end(), 0);
        for (int64_t kh = 0; kh < KH; ++kh) {
          const int64_t ih = h * stride_h - pad_top + kh * dil_h;
          if (ih < 0 || ih >= H) continue;
          for (int64_t kw = 0; kw < KW; ++kw) {
            const int64_t iw = w * stride_w - pad_left + kw * dil_w;
            if (iw < 0 || iw >= W) continue;
            const uint8_t *ip = in + ((b * H + ih) * W + iw) * C;
            const uint8_t *fp = filter + (kh * KW + kw) * C * mult_ch;
            for (int64_t c = 0; c < C; ++c) {
              const int32_t iv = static_cast<int32_t>(ip[c]) - zp_in;
              for (int64_t o = 0; o < mult_ch; ++o) {
                acc[c * mult_ch + o] +=
                    iv * (static_cast<int32_t>(fp[c * mult_ch + o]) - zp_f);
              }
            }
          }
        }
        uint8_t *op = out + ((b * Ho + h) * Wo + w) * OC;
        for (int64_t m = 0; m < OC; ++m) {
          int32_t a = acc[m] + (bias ? bias[m] : 0);
          op[m] = requant_fixed(a, multiplier, right_shift, zp_out);
        }
      }
    }
  });
  return 0;
}

int orc_dwconv_u8_nhwc_general(const uint8_t *in, const uint8_t *filter,
                               const int32_t *bias, uint8_t *out, int64_t N,
                               int64_t H, int64_t W, int64_t C,
                               int64_t mult_ch, int64_t KH, int64_t KW,
                               int stride_h, int stride_w, int dil_h,
                               int dil_w, int pad_top, int pad_left,
                               int64_t Ho, int64_t Wo, int32_t zp_in,
                               int32_t zp_f, float multiplier,
                               int32_t zp_out) {
  const int64_t OC = C * mult_ch;
  parallel_for(N * Ho, [&](int64_t rb, int64_t re) {
    for (int64_t r = rb; r < re; ++r) {
      const int64_t b = r / Ho, h = r % Ho;
      for (int64_t w = 0; w < Wo; ++w) {
        for (int64_t m = 0; m < OC; ++m) {
          const int64_t c = m / mult_ch, o = m % mult_ch;
          int32_t sum = 0;
          for (int64_t kh = 0; kh < KH; ++kh) {
            const int64_t ih = h * stride_h - pad_top + kh * dil_h;
            for (int64_t kw = 0; kw < KW; ++kw) {
              const int64_t iw = w * stride_w - pad_left + kw * dil_w;
              if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
                sum += (in[((b * H + ih) * W + iw) * C + c] - zp_in) *
                       (filter[((kh * KW + kw) * C + c) * mult_ch + o] - zp_f);
              }
            }
          }
          if (bias) sum += bias[m];
          sum = static_cast<int32_t>(std::round(sum * multiplier));
          sum += zp_out;
          out[((b * Ho + h) * Wo + w) * OC + m] =
              static_cast<uint8_t>(std::min(255, std::max(0, sum)));
        }
      }
    }
  });
  return 0;
}

int orc_avgpool_u8_nhwc(const uint8_t *in, uint8_t *out, int64_t N, int64_t H,
                        int64_t W, int64_t C, int64_t KH, int64_t KW,
                        int stride_h, int stride_w, int pad_top, int pad_left,
                        int64_t Ho, int64_t Wo) {
  int bad = 0;
  parallel_for(N * Ho, [&](int64_t rb, int64_t re) {
    std::vector<uint32_t> avg(C);
    for (int64_t r = rb; r < re; ++r) {
      const int64_t b = r / Ho, h = r % Ho;
      for (int64_t w = 0; w < Wo; ++w) {
        const int64_t hb = h * stride_h - pad_top, wb = w * stride_w - pad_left;
        const int64_t h0 = std::max<int64_t>(0, hb), w0 = std::max<int64_t>(0, wb);
        const int64_t h1 = std::min(H, hb + KH), w1 = std::min(W, wb + KW);
        const int64_t block = (h1 - h0) * (w1 - w0);
        if (block <= 0) {
          bad = 1;
          continue;
        }
        std::fill(avg.begin(), avg.end(), 0u);
        for (int64_t ih = h0; ih < h1; ++ih)
          for (int64_t iw = w0; iw < w1; ++iw) {
            const uint8_t *p = in + ((b * H + ih) * W + iw) * C;
            for (int64_t c = 0; c < C; ++c) avg[c] += p[c];
          }
        uint8_t *op = out + ((b * Ho + h) * Wo + w) * C;
        for (int64_t c = 0; c < C; ++c)
          op[c] = static_cast<uint8_t>((avg[c] + block / 2) / block);
      }
    }
  });
  return bad;
}

int orc_conv2d_f32_nchw(const float *in, const float *filter,
                        const float *bias, float *out, int64_t N, int64_t C,
                        int64_t H, int64_t W, int64_t O, int64_t KH,
                        int64_t KW, int stride_h, int stride_w, int dil_h,
                        int dil_w, int pad_top, int pad_left, int64_t Ho,
                        int64_t Wo, int act, float max_limit, float coef) {
  parallel_for(N * O, [&](int64_t rb, int64_t re) {
    for (int64_t r = rb; r < re; ++r) {
      const int64_t b = r / O, m = r % O;
      float *ob = out + (b * O + m) * Ho * Wo;
      for (int64_t h = 0; h < Ho; ++h) {
        for (int64_t w = 0; w < Wo; ++w) {
          float sum = 0;
          for (int64_t c = 0; c < C; ++c) {
            const float *ib = in + (b * C + c) * H * W;
            const float *fp = filter + (m * C + c) * KH * KW;
            for (int64_t kh = 0; kh < KH; ++kh) {
              for (int64_t kw = 0; kw < KW; ++kw) {
                const int64_t ih = -pad_top + h * stride_h + kh * dil_h;
                const int64_t iw = -pad_left + w * stride_w + kw * dil_w;
                if (ih >= 0 && ih < H && iw >= 0 && iw < W) {
                  sum += ib[ih * W + iw] * fp[kh * KW + kw];
                }
              }
            }
          }
          ob[h * Wo + w] = sum;
        }
      }
    }
  });
  bias_act_nchw(out, bias, N, O, Ho * Wo, act, max_limit, coef);
  return 0;
}

int orc_dwconv_f32_nchw(const float *in, const float *filter,
                        const float *bias, float *out, int64_t N, int64_t C,
                        int64_t H, int64_t W, int64_t mult_ch, int64_t KH,
                        int64_t KW, int stride_h, int stride_w, int dil_h,
                        int dil_w, int pad_top, int pad_left, int64_t Ho,
                        int64_t Wo, int act, float max_limit, float coef) {
  const int64_t OC = C * mult_ch;
  parallel_for(N * OC, [&](int64_t rb, int64_t re) {
    for (int64_t r = rb; r < re; ++r) {
      const int64_t b = r / OC, m = r % OC;
      const int64_t c = m / mult_ch, o = m % mult_ch;
      const float *ib = in + (b * C + c) * H * W;
      const float *fp = filter + (o * C + c) * KH * KW;
      float *ob = out + (b * OC + m) * Ho * Wo;
      for (int64_t h = 0; h < Ho; ++h) {
        for (int64_t w = 0; w < Wo; ++w) {
          float sum = 0.f;
          for (int64_t kh = 0; kh < KH; ++kh) {
            for (int64_t kw = 0; kw < KW; ++kw) {
              const int64_t ih = -pad_top + h * stride_h + kh * dil_h;
              const int64_t iw = -pad_left + w * stride_w + kw * dil_w;
              if (ih >= 0 && ih < H && iw >= 0 && iw < W)
                sum += ib[ih * W + iw] * fp[kh * KW + kw];
            }
          }
          ob[h * Wo + w] = sum;
        }
      }
    }
  });
  bias_act_nchw(out, bias, N, OC, Ho * Wo, act, max_limit, coef);
  return 0;
}

int orc_gemm_f32(const float *A, const float *B, float *C, int64_t batch,
                 int64_t M, int64_t N, int64_t K, int a_col_major,
                 int b_col_major, int c_col_major, int a_batched,
                 int b_batched) {
  for (int64_t b = 0; b < batch; ++b) {
    const float *a = A + (a_batched ? b * M * K : 0);
    const float *bm = B + (b_batched ? b * K * N : 0);
    float *c = C + b * M * N;
    parallel_for(M, [&](int64_t rb, int64_t re) {
      for (int64_t r = rb; r < re; ++r) {
        for (int64_t col = 0; col < N; ++col) {
          float sum = 0;
          for (int64_t d = 0; d < K; ++d) {
            const float av = a_col_major ? a[d * M + r] : a[r * K + d];
            const float bv = b_col_major ? bm[col * K + d] : bm[d * N + col];
            sum += av * bv;
          }
          c[c_col_major ? col * M + r : r * N + col] = sum;
        }
      }
    });
  }
  return 0;
}

int orc_gemv_f32(const float *lhs, const float *rhs, const float *bias,
                 float *out, int64_t batch, int64_t rows, int64_t K,
                 int lhs_batched, int rhs_batched) {
  for (int64_t b = 0; b < batch; ++b) {
    parallel_for(rows, [&](int64_t hb, int64_t he) {
      for (int64_t h = hb; h < he; ++h) {
        float sum = bias ? bias[h] : 0.f;
        const float *lp = lhs + (lhs_batched ? b * rows * K : 0) + h * K;
        const float *rp = rhs + (rhs_batched ? b * K : 0);
        for (int64_t w = 0; w < K; ++w) sum += lp[w] * rp[w];
        out[b * rows + h] = sum;
      }
    });
  }
  return 0;
}

// ---- Winograd ---------------------------------------------------------------

namespace {

// TransformFilter4x4 / 8x8: OIHW -> U[T][O][C]
// (mace/ops/arm/base/conv_2d_3x3_winograd.cc:237-383).
void wino_filter(const float *f, int64_t C, int64_t O, int tile, float *U) {
  const int64_t stride = O * C;
  if (tile == 2) {
    for (int64_t m = 0; m < O; ++m)
      for (int64_t c = 0; c < C; ++c) {
        const float *g = f + (m * C + c) * 9;
        float s[16];
        s[0] = g[0];
        s[1] = (g[0] + g[2] + g[1]) * 0.5f;
        s[2] = (g[0] + g[2] - g[1]) * 0.5f;
        s[3] = g[2];
        s[4] = (g[0] + g[6] + g[3]) * 0.5f;
        s[5] = ((g[0] + g[6] + g[3]) + (g[2] + g[8] + g[5]) +
                (g[1] + g[7] + g[4])) * 0.25f;
        s[6] = ((g[0] + g[6] + g[3]) + (g[2] + g[8] + g[5]) -
                (g[1] + g[7] + g[4])) * 0.25f;
        s[7] = (g[2] + g[8] + g[5]) * 0.5f;
        s[8] = (g[0] + g[6] - g[3]) * 0.5f;
        s[9] = ((g[0] + g[6] - g[3]) + (g[2] + g[8] - g[5]) +
                (g[1] + g[7] - g[4])) * 0.25f;
        s[10] = ((g[0] + g[6] - g[3]) + (g[2] + g[8] - g[5]) -
                 (g[1] + g[7] - g[4])) * 0.25f;
        s[11] = (g[2] + g[8] - g[5]) * 0.5f;
        s[12] = g[6];
        s[13] = (g[6] + g[8] + g[7]) * 0.5f;
        s[14] = (g[6] + g[8] - g[7]) * 0.5f;
        s[15] = g[8];
        for (int i = 0; i < 16; ++i) U[m * C + c + i * stride] = s[i];
      }
    return;
  }
  const float G[8][3] = {{1.0f, 0.0f, 0.0f},
                         {-2.0f / 9, -2.0f / 9, -2.0f / 9},
                         {-2.0f / 9, 2.0f / 9, -2.0f / 9},
                         {1.0f / 90, 1.0f / 45, 2.0f / 45},
                         {1.0f / 90, -1.0f / 45, 2.0f / 45},
                         {1.0f / 45, 1.0f / 90, 1.0f / 180},
                         {1.0f / 45, -1.0f / 90, 1.0f / 180},
                         {0.0f, 0.0f, 1.0f}};
  for (int64_t m = 0; m < O; ++m)
    for (int64_t c = 0; c < C; ++c) {
      const float *g = f + (m * C + c) * 9;
      float s[3][8];
      for (int i = 0; i < 8; ++i) {
        s[0][i] = g[0] * G[i][0] + g[1] * G[i][1] + g[2] * G[i][2];
        s[1][i] = g[3] * G[i][0] + g[4] * G[i][1] + g[5] * G[i][2];
        s[2][i] = g[6] * G[i][0] + g[7] * G[i][1] + g[8] * G[i][2];
      }
      for (int i = 0; i < 8; ++i)
        for (int j = 0; j < 8; ++j)
          U[m * C + c + (i * 8 + j) * stride] =
              G[i][0] * s[0][j] + G[i][1] * s[1][j] + G[i][2] * s[2][j];
    }
}

// One row/column pass of the F(6,3) input transform (the constants are double
// literals in the reference, so the products are evaluated in double).
inline void bt8(const float d[8], float o[8]) {
  o[0] = d[0] - d[6] + (d[4] - d[2]) * 5.25;
  o[7] = d[7] - d[1] + (d[3] - d[5]) * 5.25;
  float u = d[2] + d[6] - d[4] * 4.25;
  float v = d[1] + d[5] - d[3] * 4.25;
  o[1] = u + v;
  o[2] = u - v;
  u = d[6] + d[2] * 0.25 - d[4] * 1.25;
  v = d[1] * 0.5 - d[3] * 2.5 + d[5] * 2;
  o[3] = u + v;
  o[4] = u - v;
  u = d[6] + (d[2] - d[4] * 1.25) * 4;
  v = d[1] * 2 - d[3] * 2.5 + d[5] * 0.5;
  o[5] = u + v;
  o[6] = u - v;
}

inline void at8(const float d[8], float o[6]) {
  float u = d[1] + d[2];
  float v = d[1] - d[2];
  float w = d[3] + d[4];
  float x = d[3] - d[4];
  float y = d[5] + d[6];
  float z = d[5] - d[6];
  o[0] = d[0] + u + w + y * 32;
  o[1] = v + x + x + z * 16;
  o[2] = u + w * 4 + y * 8;
  o[3] = v + x * 8 + z * 4;
  o[4] = u + w * 16 + y + y;
  o[5] = v + x * 32 + z + d[7];
}

}  // namespace

int orc_conv3x3_winograd_f32_nchw(const float *in, const float *filter,
                                  const float *bias, float *out, int64_t N,
                                  int64_t C, int64_t H, int64_t W, int64_t O,
                                  int pad_top, int pad_left, int64_t Ho,
                                  int64_t Wo, int act, float max_limit,
                                  float coef, int tile_override) {
  int tile = (H > 16 && W > 16) ? 6 : 2;  // winograd.cc:41-46
  if (tile_override == 2 || tile_override == 6) tile = tile_override;
  const int in_tile = tile + 2;
  const int T = in_tile * in_tile;
  const int64_t pHo = (Ho + tile - 1) / tile * tile;
  const int64_t pWo = (Wo + tile - 1) / tile * tile;
  // CalOutputShapeAndPadSize, mace/ops/arm/base/conv_2d.cc:79-120: the padded
  // input covers the padded output (stride 1, 3x3).
  const int64_t pH = pHo + 2, pW = pWo + 2;
  const int64_t th = pHo / tile, tw = pWo / tile, tiles = th * tw;

  std::vector<float> pin(static_cast<size_t>(N) * C * pH * pW, 0.f);
  for (int64_t nc = 0; nc < N * C; ++nc)
    for (int64_t h = 0; h < H; ++h) {
      if (h + pad_top >= pH) continue;
      const int64_t wcopy = std::min<int64_t>(W, pW - pad_left);
      std::memcpy(&pin[(nc * pH + h + pad_top) * pW + pad_left],
                  in + (nc * H + h) * W, sizeof(float) * wcopy);
    }
  std::vector<float> U(static_cast<size_t>(T) * O * C);
  wino_filter(filter, C, O, tile, U.data());
  std::vector<float> V(static_cast<size_t>(N) * T * C * tiles);
  std::vector<float> Mx(static_cast<size_t>(N) * T * O * tiles);
  std::vector<float> pout(static_cast<size_t>(N) * O * pHo * pWo);

  // input transform: NCHW -> V[N][T][C][tiles]
  const int64_t vstride = C * tiles;
  parallel_for(N * C, [&](int64_t rb, int64_t re) {
    for (int64_t r = rb; r < re; ++r) {
      const int64_t n = r / C, c = r % C;
      int64_t ti = 0;
      for (int64_t h = 0; h < pH - 2; h += tile)
        for (int64_t w = 0; w < pW - 2; w += tile, ++ti) {
          const float *ip = &pin[((n * C + c) * pH + h) * pW + w];
          float *op = &V[n * T * vstride + c * tiles + ti];
          if (tile == 2) {
            float d[16];
            for (int i = 0; i < 4; ++i)
              for (int j = 0; j < 4; ++j) d[i * 4 + j] = ip[i * pW + j];
            float s[16];
            s[0] = (d[0] - d[8]) - (d[2] - d[10]);
            s[1] = (d[1] - d[9]) + (d[2] - d[10]);
            s[2] = (d[2] - d[10]) - (d[1] - d[9]);
            s[3] = (d[1] - d[9]) - (d[3] - d[11]);
            s[4] = (d[4] + d[8]) - (d[6] + d[10]);
            s[5] = (d[5] + d[9]) + (d[6] + d[10]);
            s[6] = (d[6] + d[10]) - (d[5] + d[9]);
            s[7] = (d[5] + d[9]) - (d[7] + d[11]);
            s[8] = (d[8] - d[4]) - (d[10] - d[6]);
            s[9] = (d[9] - d[5]) + (d[10] - d[6]);
            s[10] = (d[10] - d[6]) - (d[9] - d[5]);
            s[11] = (d[9] - d[5]) - (d[11] - d[7]);
            s[12] = (d[4] - d[12]) - (d[6] - d[14]);
            s[13] = (d[5] - d[13]) + (d[6] - d[14]);
            s[14] = (d[6] - d[14]) - (d[5] - d[13]);
            s[15] = (d[5] - d[13]) - (d[7] - d[15]);
            for (int i = 0; i < 16; ++i) op[i * vstride] = s[i];
          } else {
            float s[8][8];
            for (int i = 0; i < 8; ++i) {
              float d[8];
              for (int j = 0; j < 8; ++j) d[j] = ip[i * pW + j];
              bt8(d, s[i]);
            }
            for (int i = 0; i < 8; ++i) {
              float d[8], o[8];
              for (int j = 0; j < 8; ++j) d[j] = s[j][i];
              bt8(d, o);
              // row order of the second pass: 0, 8.., 16.., 24.., ..., 56..
              for (int j = 0; j < 8; ++j) op[(j * 8 + i) * vstride] = o[j];
            }
          }
        }
    }
  });

  // batched GEMM per image: M[t] = U[t] (O x C) * V[t] (C x tiles), float
  // accumulation, depth ascending.
  parallel_for(N * T, [&](int64_t rb, int64_t re) {
    for (int64_t r = rb; r < re; ++r) {
      const int64_t n = r / T, t = r % T;
      const float *u = &U[t * O * C];
      const float *v = &V[(n * T + t) * C * tiles];
      float *m = &Mx[(n * T + t) * O * tiles];
      for (int64_t o = 0; o < O; ++o) {
        float *mr = m + o * tiles;
        for (int64_t j = 0; j < tiles; ++j) mr[j] = 0.f;
        for (int64_t c = 0; c < C; ++c) {
          const float uv = u[o * C + c];
          const float *vr = v + c * tiles;
          for (int64_t j = 0; j < tiles; ++j) mr[j] += uv * vr[j];
        }
      }
    }
  });

  // output transform: M[N][T][O][tiles] -> padded NCHW
  const int64_t mstride = O * tiles;
  parallel_for(N * O, [&](int64_t rb, int64_t re) {
    for (int64_t r = rb; r < re; ++r) {
      const int64_t n = r / O, m = r % O;
      int64_t ti = 0;
      for (int64_t h = 0; h < pHo; h += tile)
        for (int64_t w = 0; w < pWo; w += tile, ++ti) {
          const float *ip = &Mx[n * T * mstride + m * tiles + ti];
          float *op = &pout[((n * O + m) * pHo + h) * pWo + w];
          if (tile == 2) {
            float d[16];
            for (int i = 0; i < 16; ++i) d[i] = ip[i * mstride];
            float s0 = d[0] + d[1] + d[2], s1 = d[1] - d[2] - d[3];
            float s2 = d[4] + d[5] + d[6], s3 = d[5] - d[6] - d[7];
            float s4 = d[8] + d[9] + d[10], s5 = d[9] - d[10] - d[11];
            float s6 = d[12] + d[13] + d[14], s7 = d[13] - d[14] - d[15];
            op[0] = s0 + s2 + s4;
            op[1] = s1 + s3 + s5;
            op[pWo] = s2 - s4 - s6;
            op[pWo + 1] = s3 - s5 - s7;
          } else {
            float s[8][6];
            for (int i = 0; i < 8; ++i) {
              float d[8];
              for (int j = 0; j < 8; ++j) d[j] = ip[(i * 8 + j) * mstride];
              at8(d, s[i]);
            }
            for (int i = 0; i < 6; ++i) {
              float d[8], o[6];
              for (int j = 0; j < 8; ++j) d[j] = s[j][i];
              at8(d, o);
              for (int j = 0; j < 6; ++j) op[j * pWo + i] = o[j];
            }
          }
        }
    }
  });

  // UnPadOutput
  for (int64_t no = 0; no < N * O; ++no)
    for (int64_t h = 0; h < Ho; ++h)
      std::memcpy(out + (no * Ho + h) * Wo, &pout[(no * pHo + h) * pWo],
                  sizeof(float) * Wo);
  bias_act_nchw(out, bias, N, O, Ho * Wo, act, max_limit, coef);
  return 0;
}

int orc_pooling_f32_nchw(const float *in, float *out, int64_t N, int64_t C, int64_t H, int64_t W,
                         int64_t KH, int64_t KW, int stride_h, int stride_w, int dil_h, int dil_w,
                         int pad_top, int pad_left, int64_t Ho, int64_t Wo, int pooling_type) {
  if (pooling_type != 1 && pooling_type != 2) return 1;
  parallel_for(N * C, [&](int64_t pb, int64_t pe) {
    for (int64_t pl = pb; pl < pe; ++pl) {
      const float *ip = in + pl * H * W;
      float *op = out + pl * Ho * Wo;
      for (int64_t h = 0; h < Ho; ++h)
        for (int64_t w = 0; w < Wo; ++w) {
          // MaxPooling: res = lowest(), max over in-bounds taps (pooling.cc:150-170);
          // AvgPooling: sum over in-bounds taps / their count (pooling.cc:213-236)
          float res = pooling_type == 2 ? std::numeric_limits<float>::lowest() : 0.f;
          int block_size = 0;
          for (int64_t fh = 0; fh < KH; ++fh)
            for (int64_t fw = 0; fw < KW; ++fw) {
              const int64_t inh = h * stride_h + dil_h * fh - pad_top;
              const int64_t inw = w * stride_w + dil_w * fw - pad_left;
              if (inh < 0 || inh >= H || inw < 0 || inw >= W) continue;
              const float v = ip[inh * W + inw];
              if (pooling_type == 2) res = std::max(res, v);
              else res += v;
              ++block_size;
            }
          if (pooling_type == 1) res = block_size > 0 ? res / block_size : 0.f;
          op[h * Wo + w] = res;
        }
    }
  });
  return 0;
}

int orc_eltwise_f32(const float *in0, const float *in1, float *out, int64_t size, int type,
                    float scalar_input, int has_coeff, float coeff0, float coeff1, int swapped) {
  // TensorEltwise / TensorScalarEltwise (mace/ops/eltwise.cc:419-700); in1 == NULL is the
  // tensor-scalar form.
  float c0 = coeff0, c1 = coeff1;
  if (swapped && type == 0) std::swap(c0, c1);
  for (int64_t i = 0; i < size; ++i) {
    const float a = in0[i], b = in1 != nullptr ? in1[i] : scalar_input;
    float r;
    switch (type) {
      case 0: {
        if (has_coeff) {
          volatile float p0 = a * c0, p1 = b * c1;  // two rounded products, then the sum
          r = p0 + p1;
        } else {
          r = a + b;
        }
        break;
      }
      case 1: r = swapped ? b - a : a - b; break;
      case 2: r = a * b; break;
      case 3: r = swapped ? b / a : a / b; break;
      case 4: r = std::min(a, b); break;
      case 5: r = std::max(a, b); break;
      case 6: r = -a; break;
      case 7: r = std::fabs(a); break;
      case 8: r = std::pow(a - b, 2.f); break;
      case 12: r = std::fmax(coeff0, std::fmin(coeff1, a)); break;
      default: return 1;
    }
    out[i] = r;
  }
  return 0;
}

int orc_activation_f32(const float *in, float *out, int64_t size, int act, float max_limit, float coef) {
  for (int64_t i = 0; i < size; ++i) out[i] = activate(in[i], act, max_limit, coef);
  return 0;
}

int orc_softmax_f32(const float *in, float *out, int64_t outer, int64_t classes, int64_t inner, int use_log) {
  // SoftmaxOp<RT_CPU,float> (mace/ops/softmax.cc:76-290): per position the maximum over the
  // classes, exp(x - max), the sum in class order, the division, then log if asked.
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const float *ip = in + o * classes * inner + i;
      float *op = out + o * classes * inner + i;
      float mx = std::numeric_limits<float>::lowest();
      for (int64_t c = 0; c < classes; ++c) mx = std::max(mx, ip[c * inner]);
      float sum = 0.f;
      for (int64_t c = 0; c < classes; ++c) {
        op[c * inner] = std::exp(ip[c * inner] - mx);
        sum += op[c * inner];
      }
      for (int64_t c = 0; c < classes; ++c) {
        op[c * inner] /= sum;
        if (use_log) op[c * inner] = std::log(op[c * inner]);
      }
    }
  return 0;
}

void orc_dequantize_u8(const uint8_t *in, int64_t n, float scale, int32_t zero_point, float *out) {
  // QuantizeUtil::Dequantize (mace/core/quantize.h:187-197)
  for (int64_t i = 0; i < n; ++i) out[i] = scale * (in[i] - zero_point);
}

void orc_dequantize_i32(const int32_t *in, int64_t n, float scale, int32_t zero_point, float *out) {
  for (int64_t i = 0; i < n; ++i) out[i] = scale * (in[i] - zero_point);
}

}  // extern "C"
