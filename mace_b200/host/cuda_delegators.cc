// CUDA implementations of the hot-path delegators.  Each Compute body does the
// host work that the corresponding CPU operator does before it reaches its
// arithmetic kernel (shapes, Resize, bias rescale, multiplier derivation) and
// then makes one call into the device library's C ABI.
#include <cmath>
#include <cstring>
#include <memory>
#include <vector>

#include "delegators.h"

namespace mace {

CudaRuntime::~CudaRuntime() {
  if (ctx_ != nullptr) mb_destroy(ctx_);
}

MaceStatus CudaRuntime::Init(int device) {
  const int rc = mb_init(device, &ctx_);
  if (rc != MB_SUCCESS) {
    return MaceStatus(static_cast<MaceStatus::Code>(rc), "mb_init failed: no sm_100a CUDA device");
  }
  return MaceStatus::MACE_SUCCESS;
}

MaceStatus CudaRuntime::New(size_t bytes, void **ptr) { return Status(mb_malloc(ctx_, bytes, ptr)); }

void CudaRuntime::Delete(void *ptr) { mb_free(ctx_, ptr); }

MaceStatus CudaRuntime::Status(int rc) const {
  if (rc == MB_SUCCESS) return MaceStatus::MACE_SUCCESS;
  return MaceStatus(static_cast<MaceStatus::Code>(rc), mb_last_error(ctx_));
}

namespace ops {
namespace cuda {
namespace q8 {

// GetBiasData for a device-resident bias (mace/ops/arm/q8/quantization_util.cc:20-46):
// a null bias means "no bias" to the kernels; a bias whose scale differs from
// input_scale * filter_scale by more than 1e-6 is rescaled with
// round(bias * bias_scale / (input_scale * filter_scale)).  The rescaled copy
// is kept while the bias tensor and scales stay the same (weights are constant).
class BiasCache {
 public:
  MaceStatus Get(CudaRuntime *rt, const Tensor *bias, float input_scale, float filter_scale,
                 index_t channels, const int32_t **out) {
    if (bias == nullptr) {
      *out = nullptr;
      return MaceStatus::MACE_SUCCESS;
    }
    MACE_CHECK(bias->size() >= channels);
    const bool adjust = std::fabs(input_scale * filter_scale - bias->scale()) > 1e-6;
    if (!adjust) {
      *out = bias->memory<int32_t>();
      return MaceStatus::MACE_SUCCESS;
    }
    if (adjusted_ == nullptr || src_ != bias || in_scale_ != input_scale || f_scale_ != filter_scale) {
      std::vector<int32_t> host(static_cast<size_t>(channels));
      MACE_RETURN_IF_ERROR(rt->Status(mb_memcpy_d2h(rt->ctx(), host.data(), bias->memory<int32_t>(),
                                                    sizeof(int32_t) * channels)));
      MACE_RETURN_IF_ERROR(rt->Status(mb_stream_sync(rt->ctx())));
      const float adjust_scale = bias->scale() / (input_scale * filter_scale);
      for (auto &v : host) v = static_cast<int32_t>(roundf(v * adjust_scale));
      adjusted_ = std::make_unique<Tensor>(rt, DT_INT32, std::vector<index_t>{channels}, true);
      MACE_RETURN_IF_ERROR(rt->Status(mb_memcpy_h2d(rt->ctx(), adjusted_->mutable_memory<int32_t>(),
                                                    host.data(), sizeof(int32_t) * channels)));
      MACE_RETURN_IF_ERROR(rt->Status(mb_stream_sync(rt->ctx())));
      src_ = bias;
      in_scale_ = input_scale;
      f_scale_ = filter_scale;
    }
    *out = adjusted_->memory<int32_t>();
    return MaceStatus::MACE_SUCCESS;
  }

 private:
  std::unique_ptr<Tensor> adjusted_;
  const Tensor *src_ = nullptr;
  float in_scale_ = 0.f, f_scale_ = 0.f;
};

// uint8 GEMM: the arithmetic of MatMulFixpointImpl (mace/ops/matmul.cc:228-394).
// A uint8 output is requantized with the fixed-point multiplier of
// (lhs scale * rhs scale / output scale); an int32 output receives the raw
// accumulators and gets scale = lhs scale * rhs scale, zero point 0.
class Gemm : public delegator::Gemm {
 public:
  explicit Gemm(const delegator::GemmParam &param) : delegator::Gemm(param) {}

  MaceStatus Compute(const OpContext *context, const Tensor *lhs, const Tensor *rhs,
                     const index_t batch, const index_t rows, const index_t cols,
                     const index_t depth, const MatrixMajor lhs_major, const MatrixMajor rhs_major,
                     const MatrixMajor output_major, const bool lhs_batched,
                     const bool rhs_batched, Tensor *output) override {
    CudaRuntime *rt = CudaRuntimeOf(context);
    const bool out_int32 = output->dtype() == DT_INT32;
    int32_t multiplier = 1 << 30;
    int right_shift = 0;
    if (out_int32) {
      output->SetScale(lhs->scale() * rhs->scale());
      output->SetZeroPoint(0);
    } else {
      MACE_RETURN_IF_ERROR(GetOutputMultiplierAndShift(lhs->scale(), rhs->scale(), output->scale(),
                                                       &multiplier, &right_shift));
    }
    return rt->Status(mb_gemm_u8(
        rt->ctx(), lhs->memory<uint8_t>(), rhs->memory<uint8_t>(), nullptr,
        output->mutable_memory<void>(), out_int32 ? 1 : 0, batch, rows, cols, depth,
        lhs_major == ColMajor, rhs_major == ColMajor, output_major == ColMajor, lhs_batched,
        rhs_batched, lhs->zero_point(), rhs->zero_point(), multiplier, right_shift,
        output->zero_point(), 0));
  }

  MaceStatus Compute(const OpContext *context, const Tensor *lhs, const Tensor *rhs,
                     const index_t batch, const index_t lhs_rows, const index_t lhs_cols,
                     const index_t rhs_rows, const index_t rhs_cols, const bool transpose_lhs,
                     const bool transpose_rhs, const bool transpose_out, const bool lhs_batched,
                     const bool rhs_batched, Tensor *output) override {
    // Same mapping as the reference's transpose overloads (mace/ops/ref/gemm.cc:108-150):
    // a transposed row-major matrix is the column-major matrix of the swapped shape.
    const index_t rows = transpose_lhs ? lhs_cols : lhs_rows;
    const index_t depth = transpose_lhs ? lhs_rows : lhs_cols;
    const index_t cols = transpose_rhs ? rhs_rows : rhs_cols;
    const index_t rhs_depth = transpose_rhs ? rhs_cols : rhs_rows;
    MACE_CHECK(depth == rhs_depth);
    return Compute(context, lhs, rhs, batch, rows, cols, depth,
                   transpose_lhs ? ColMajor : RowMajor, transpose_rhs ? ColMajor : RowMajor,
                   transpose_out ? ColMajor : RowMajor, lhs_batched, rhs_batched, output);
  }
};

// uint8 GEMV with the float multiplier rule of arm::q8::Gemv
// (mace/ops/arm/q8/gemv.cc:36-171).
class Gemv : public delegator::Gemv {
 public:
  explicit Gemv(const DelegatorParam &param) : delegator::Gemv(param) {}

  MaceStatus Compute(const OpContext *context, const Tensor *lhs, const Tensor *rhs,
                     const Tensor *bias, const index_t batch, const index_t lhs_height,
                     const index_t lhs_width, const bool lhs_batched, const bool rhs_batched,
                     Tensor *output) override {
    CudaRuntime *rt = CudaRuntimeOf(context);
    const bool out_int32 = output->dtype() == DT_INT32;
    float multiplier = 0.f;
    if (!out_int32) {
      if (!(output->scale() > 0))
        return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "output scale must not be zero");
      multiplier = lhs->scale() * rhs->scale() / output->scale();
    }
    mb_set_option(rt->ctx(), "gemv_lhs_const", lhs->is_weight() ? 1 : 0);
    return rt->Status(mb_gemv_u8(rt->ctx(), lhs->memory<uint8_t>(), rhs->memory<uint8_t>(),
                                 bias ? bias->memory<int32_t>() : nullptr,
                                 output->mutable_memory<void>(), out_int32 ? 1 : 0, batch,
                                 lhs_height, lhs_width, lhs_batched, rhs_batched,
                                 lhs->zero_point(), rhs->zero_point(), multiplier,
                                 output->zero_point(), /*add_zp_out=*/1));
  }
};

// uint8 Conv2D, NHWC x OHWI: everything Conv2dOp<RT_CPU,uint8_t>::Run does
// before its GEMM (mace/ops/conv_2d.cc:201-310), then mb_conv2d_u8_nhwc.
class Conv2d : public delegator::Conv2d {
 public:
  explicit Conv2d(const delegator::Conv2dParam &param) : delegator::Conv2d(param) {}

  MaceStatus Compute(const OpContext *context, const Tensor *input, const Tensor *filter,
                     Tensor *output) override {
    CudaRuntime *rt = CudaRuntimeOf(context);
    if (dilations_[0] != 1 || dilations_[1] != 1)
      return MaceStatus(MaceStatus::MACE_UNSUPPORTED,
                        "Quantization convolution does not support dilation > 1 yet.");
    MACE_CHECK(input->dim_size() == 4 && filter->dim_size() == 4);
    index_t out_h = 0, out_w = 0;
    std::vector<int> paddings(2);
    if (paddings_.empty()) {
      MACE_RETURN_IF_ERROR(CalcPaddingAndOutputSize(input->dim(1), input->dim(2), filter->dim(1),
                                                    filter->dim(2), dilations_.data(),
                                                    strides_.data(), padding_type_, &out_h, &out_w,
                                                    paddings.data()));
    } else {
      paddings = paddings_;
      CalcOutputSize(input->dim(1), input->dim(2), filter->dim(1), filter->dim(2), paddings.data(),
                     dilations_.data(), strides_.data(), FLOOR, &out_h, &out_w);
    }
    const index_t channels = filter->dim(0);
    MACE_CHECK(filter->dim(3) == input->dim(3));
    MACE_RETURN_IF_ERROR(output->Resize({input->dim(0), out_h, out_w, channels}));
    const int32_t *bias_data = nullptr;
    MACE_RETURN_IF_ERROR(
        bias_cache_.Get(rt, bias_, input->scale(), filter->scale(), channels, &bias_data));
    int32_t multiplier = 0;
    int right_shift = 0;
    // Pipeline::Make(bias, channels, filter scale, input scale, output scale, zp)
    MACE_RETURN_IF_ERROR(GetOutputMultiplierAndShift(filter->scale(), input->scale(),
                                                     output->scale(), &multiplier, &right_shift));
    // weights (Tensor::is_weight(), mace/core/tensor.h) are not written by the work enqueued ahead of
    // this call, so a kernel may read them while its predecessor still runs
    mb_set_option(rt->ctx(), "conv_filter_const",
                  filter->is_weight() && (bias_ == nullptr || bias_->is_weight()) ? 1 : 0);
    return rt->Status(mb_conv2d_u8_nhwc(
        rt->ctx(), input->memory<uint8_t>(), filter->memory<uint8_t>(), bias_data,
        output->mutable_memory<uint8_t>(), input->dim(0), input->dim(1), input->dim(2),
        input->dim(3), channels, filter->dim(1), filter->dim(2), strides_[0], strides_[1],
        paddings[0] >> 1, paddings[1] >> 1, out_h, out_w, input->zero_point(),
        filter->zero_point(), multiplier, right_shift, output->zero_point()));
  }

 private:
  BiasCache bias_cache_;
};

// uint8 DepthwiseConv2d, NHWC x HWIM (mace/ops/depthwise_conv2d.cc:152-250).
class DepthwiseConv2d : public delegator::DepthwiseConv2d {
 public:
  explicit DepthwiseConv2d(const delegator::DepthwiseConv2dParam &param)
      : delegator::DepthwiseConv2d(param) {}

  MaceStatus Compute(const OpContext *context, const Tensor *input, const Tensor *filter,
                     Tensor *output) override {
    CudaRuntime *rt = CudaRuntimeOf(context);
    MACE_CHECK(input->dim_size() == 4 && filter->dim_size() == 4);
    MACE_CHECK(filter->dim(2) == input->dim(3));
    index_t out_h = 0, out_w = 0;
    std::vector<int> paddings(2);
    if (paddings_.empty()) {
      MACE_RETURN_IF_ERROR(CalcPaddingAndOutputSize(input->dim(1), input->dim(2), filter->dim(0),
                                                    filter->dim(1), dilations_.data(),
                                                    strides_.data(), padding_type_, &out_h, &out_w,
                                                    paddings.data()));
    } else {
      paddings = paddings_;
      CalcOutputSize(input->dim(1), input->dim(2), filter->dim(0), filter->dim(1), paddings.data(),
                     dilations_.data(), strides_.data(), FLOOR, &out_h, &out_w);
    }
    const index_t out_channels = filter->dim(2) * filter->dim(3);
    MACE_RETURN_IF_ERROR(output->Resize({input->dim(0), out_h, out_w, out_channels}));
    const int32_t *bias_data = nullptr;
    MACE_RETURN_IF_ERROR(
        bias_cache_.Get(rt, bias_, input->scale(), filter->scale(), out_channels, &bias_data));
    const bool dilated = dilations_[0] != 1 || dilations_[1] != 1;
    int32_t multiplier = 1 << 30;
    int right_shift = 0;
    float multiplier_f = 0.f;
    if (dilated) {
      multiplier_f = input->scale() * filter->scale() / output->scale();
    } else {
      MACE_RETURN_IF_ERROR(GetOutputMultiplierAndShift(input->scale(), filter->scale(),
                                                       output->scale(), &multiplier, &right_shift));
    }
    // Constant filter and bias: keep the fast path's tap words from call to call, as the CPU
    // Winograd delegator keeps its transformed filter (conv_2d_3x3_winograd.cc:120-145).
    const void *prepacked = nullptr;
    const bool constant = filter->is_weight() && (bias_ == nullptr || bias_->is_weight());
    const size_t packed_bytes = mb_dwconv3x3_u8_prepacked_bytes(out_channels);
    if (constant && !dilated && filter->dim(0) == 3 && filter->dim(1) == 3 && filter->dim(3) == 1 &&
        packed_bytes > 0 && input->zero_point() >= 0 && input->zero_point() <= 255 &&
        filter->zero_point() >= 0 && filter->zero_point() <= 255) {
      if (packed_ == nullptr || packed_filter_ != filter || packed_bias_ != bias_data ||
          packed_zp_in_ != input->zero_point() || packed_zp_f_ != filter->zero_point()) {
        packed_ = std::make_unique<Tensor>(
            rt, DT_UINT8, std::vector<index_t>{static_cast<index_t>(packed_bytes)}, true);
        MACE_RETURN_IF_ERROR(rt->Status(mb_dwconv3x3_u8_prepack(
            rt->ctx(), filter->memory<uint8_t>(), bias_data, out_channels, input->zero_point(),
            filter->zero_point(), packed_->mutable_memory<uint8_t>())));
        packed_filter_ = filter;
        packed_bias_ = bias_data;
        packed_zp_in_ = input->zero_point();
        packed_zp_f_ = filter->zero_point();
      }
      prepacked = packed_->memory<uint8_t>();
    }
    return rt->Status(mb_dwconv_u8_nhwc_prepacked(
        rt->ctx(), input->memory<uint8_t>(), filter->memory<uint8_t>(), bias_data, prepacked,
        output->mutable_memory<uint8_t>(), input->dim(0), input->dim(1), input->dim(2),
        input->dim(3), filter->dim(3), filter->dim(0), filter->dim(1), strides_[0], strides_[1],
        dilations_[0], dilations_[1], paddings[0] >> 1, paddings[1] >> 1, out_h, out_w,
        input->zero_point(), filter->zero_point(), multiplier, right_shift, output->zero_point(),
        dilated ? 1 : 0, multiplier_f));
  }

 private:
  BiasCache bias_cache_;
  std::unique_ptr<Tensor> packed_;
  const Tensor *packed_filter_ = nullptr;
  const int32_t *packed_bias_ = nullptr;
  int32_t packed_zp_in_ = 0, packed_zp_f_ = 0;
};

}  // namespace q8

namespace fp32 {

// Conv shape bookkeeping shared by the fp32 convolution delegators: NCHW input,
// OIHW filter (CalcNCHWPaddingAndOutputSize, mace/ops/ref/conv_2d.cc:46-66).
struct ConvGeometry {
  index_t out_h = 0, out_w = 0;
  int pad_top = 0, pad_left = 0;
};

static MaceStatus Geometry(const Tensor *input, index_t k_h, index_t k_w,
                           const std::vector<int> &strides, const std::vector<int> &dilations,
                           const std::vector<int> &paddings_in, Padding padding_type,
                           ConvGeometry *g) {
  std::vector<int> paddings(2);
  if (paddings_in.empty()) {
    MACE_RETURN_IF_ERROR(CalcPaddingAndOutputSize(input->dim(2), input->dim(3), k_h, k_w,
                                                  dilations.data(), strides.data(), padding_type,
                                                  &g->out_h, &g->out_w, paddings.data()));
  } else {
    paddings = paddings_in;
    CalcOutputSize(input->dim(2), input->dim(3), k_h, k_w, paddings.data(), dilations.data(),
                   strides.data(), FLOOR, &g->out_h, &g->out_w);
  }
  g->pad_top = paddings[0] >> 1;
  g->pad_left = paddings[1] >> 1;
  return MaceStatus::MACE_SUCCESS;
}

class Gemm : public delegator::Gemm {
 public:
  explicit Gemm(const delegator::GemmParam &param) : delegator::Gemm(param) {}
  MaceStatus Compute(const OpContext *context, const Tensor *lhs, const Tensor *rhs,
                     const index_t batch, const index_t rows, const index_t cols,
                     const index_t depth, const MatrixMajor lhs_major, const MatrixMajor rhs_major,
                     const MatrixMajor output_major, const bool lhs_batched,
                     const bool rhs_batched, Tensor *output) override {
    CudaRuntime *rt = CudaRuntimeOf(context);
    return rt->Status(mb_gemm_f32(rt->ctx(), lhs->memory<float>(), rhs->memory<float>(),
                                  output->mutable_memory<float>(), batch, rows, cols, depth,
                                  lhs_major == ColMajor, rhs_major == ColMajor,
                                  output_major == ColMajor, lhs_batched, rhs_batched));
  }
  MaceStatus Compute(const OpContext *context, const Tensor *lhs, const Tensor *rhs,
                     const index_t batch, const index_t lhs_rows, const index_t lhs_cols,
                     const index_t rhs_rows, const index_t rhs_cols, const bool transpose_lhs,
                     const bool transpose_rhs, const bool transpose_out, const bool lhs_batched,
                     const bool rhs_batched, Tensor *output) override {
    const index_t rows = transpose_lhs ? lhs_cols : lhs_rows;
    const index_t depth = transpose_lhs ? lhs_rows : lhs_cols;
    const index_t cols = transpose_rhs ? rhs_rows : rhs_cols;
    MACE_CHECK(depth == (transpose_rhs ? rhs_cols : rhs_rows));
    return Compute(context, lhs, rhs, batch, rows, cols, depth,
                   transpose_lhs ? ColMajor : RowMajor, transpose_rhs ? ColMajor : RowMajor,
                   transpose_out ? ColMajor : RowMajor, lhs_batched, rhs_batched, output);
  }
};

class Gemv : public delegator::Gemv {
 public:
  explicit Gemv(const DelegatorParam &param) : delegator::Gemv(param) {}
  MaceStatus Compute(const OpContext *context, const Tensor *lhs, const Tensor *rhs,
                     const Tensor *bias, const index_t batch, const index_t lhs_height,
                     const index_t lhs_width, const bool lhs_batched, const bool rhs_batched,
                     Tensor *output) override {
    CudaRuntime *rt = CudaRuntimeOf(context);
    return rt->Status(mb_gemv_f32(rt->ctx(), lhs->memory<float>(), rhs->memory<float>(),
                                  bias ? bias->memory<float>() : nullptr,
                                  output->mutable_memory<float>(), batch, lhs_height, lhs_width,
                                  lhs_batched, rhs_batched));
  }
};

// General direct convolution and the 1x1-as-GEMM route (the library picks).
class Conv2d : public delegator::Conv2d {
 public:
  explicit Conv2d(const delegator::Conv2dParam &param) : delegator::Conv2d(param) {}
  MaceStatus Compute(const OpContext *context, const Tensor *input, const Tensor *filter,
                     Tensor *output) override {
    CudaRuntime *rt = CudaRuntimeOf(context);
    MACE_CHECK(input->dim(1) == filter->dim(1));
    ConvGeometry g;
    MACE_RETURN_IF_ERROR(Geometry(input, filter->dim(2), filter->dim(3), strides_, dilations_,
                                  paddings_, padding_type_, &g));
    MACE_RETURN_IF_ERROR(output->Resize({input->dim(0), filter->dim(0), g.out_h, g.out_w}));
    if (residual_ != nullptr && residual_->size() != output->size())
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "residual and convolution output differ in size");
    return rt->Status(mb_conv2d_f32_nchw_residual(
        rt->ctx(), input->memory<float>(), filter->memory<float>(),
        bias_ ? bias_->memory<float>() : nullptr, residual_ ? residual_->memory<float>() : nullptr,
        output->mutable_memory<float>(), input->dim(0), input->dim(1), input->dim(2), input->dim(3),
        filter->dim(0), filter->dim(2), filter->dim(3), strides_[0], strides_[1], dilations_[0],
        dilations_[1], g.pad_top, g.pad_left, g.out_h, g.out_w, activation_, max_limit_, coefficient_));
  }
  bool SetResidual(const Tensor *residual) override {
    residual_ = residual;
    return true;
  }

 private:
  const Tensor *residual_ = nullptr;
};

// 3x3 stride-1 Winograd; the transformed filter is cached while the filter is a
// weight, as the CPU delegator does (conv_2d_3x3_winograd.cc:120-145).
class Conv2dK3x3Winograd : public delegator::Conv2d {
 public:
  explicit Conv2dK3x3Winograd(const delegator::Conv2dParam &param) : delegator::Conv2d(param) {}
  MaceStatus Compute(const OpContext *context, const Tensor *input, const Tensor *filter,
                     Tensor *output) override {
    CudaRuntime *rt = CudaRuntimeOf(context);
    MACE_CHECK(filter->dim(2) == 3 && filter->dim(3) == 3 && strides_[0] == 1 && strides_[1] == 1 &&
               dilations_[0] == 1 && dilations_[1] == 1);
    ConvGeometry g;
    MACE_RETURN_IF_ERROR(Geometry(input, 3, 3, strides_, dilations_, paddings_, padding_type_, &g));
    MACE_RETURN_IF_ERROR(output->Resize({input->dim(0), filter->dim(0), g.out_h, g.out_w}));
    const int tile = (input->dim(2) > 16 && input->dim(3) > 16) ? 6 : 2;
    const float *transformed = nullptr;
    if (filter->is_weight()) {
      if (transformed_filter_ == nullptr || tile != out_tile_size_ || src_ != filter) {
        const index_t t = (tile + 2) * (tile + 2);
        transformed_filter_ = std::make_unique<Tensor>(
            rt, DT_FLOAT, std::vector<index_t>{t, filter->dim(0), filter->dim(1)}, true);
        MACE_RETURN_IF_ERROR(rt->Status(mb_winograd_transform_filter_f32(
            rt->ctx(), filter->memory<float>(), transformed_filter_->mutable_memory<float>(),
            filter->dim(1), filter->dim(0), tile)));
        out_tile_size_ = tile;
        src_ = filter;
      }
      transformed = transformed_filter_->memory<float>();
    }
    return rt->Status(mb_conv3x3_winograd_f32_nchw(
        rt->ctx(), input->memory<float>(), filter->memory<float>(), transformed,
        bias_ ? bias_->memory<float>() : nullptr, output->mutable_memory<float>(), input->dim(0),
        input->dim(1), input->dim(2), input->dim(3), filter->dim(0), g.pad_top, g.pad_left,
        g.out_h, g.out_w, activation_, max_limit_, coefficient_, tile));
  }

 private:
  std::unique_ptr<Tensor> transformed_filter_;
  int out_tile_size_ = 0;
  const Tensor *src_ = nullptr;
};

// fp32 depthwise, NCHW, filter [multiplier, C, kh, kw].
class DepthwiseConv2d : public delegator::DepthwiseConv2d {
 public:
  explicit DepthwiseConv2d(const delegator::DepthwiseConv2dParam &param)
      : delegator::DepthwiseConv2d(param) {}
  MaceStatus Compute(const OpContext *context, const Tensor *input, const Tensor *filter,
                     Tensor *output) override {
    CudaRuntime *rt = CudaRuntimeOf(context);
    MACE_CHECK(input->dim(1) == filter->dim(1));
    ConvGeometry g;
    MACE_RETURN_IF_ERROR(Geometry(input, filter->dim(2), filter->dim(3), strides_, dilations_,
                                  paddings_, padding_type_, &g));
    MACE_RETURN_IF_ERROR(
        output->Resize({input->dim(0), filter->dim(0) * filter->dim(1), g.out_h, g.out_w}));
    return rt->Status(mb_dwconv_f32_nchw(
        rt->ctx(), input->memory<float>(), filter->memory<float>(),
        bias_ ? bias_->memory<float>() : nullptr, output->mutable_memory<float>(), input->dim(0),
        input->dim(1), input->dim(2), input->dim(3), filter->dim(0), filter->dim(2),
        filter->dim(3), strides_[0], strides_[1], dilations_[0], dilations_[1], g.pad_top,
        g.pad_left, g.out_h, g.out_w, activation_, max_limit_, coefficient_));
  }
};

}  // namespace fp32
}  // namespace cuda

void RegisterAllCudaOpDelegators(OpDelegatorRegistry *registry) {
  MACE_REGISTER_DELEGATOR(registry, cuda::q8::Gemm, delegator::GemmParam,
                          MACE_DELEGATOR_KEY(Gemm, RuntimeType::RT_CUDA, uint8_t, ImplType::CUDA));
  MACE_REGISTER_DELEGATOR(registry, cuda::q8::Gemv, DelegatorParam,
                          MACE_DELEGATOR_KEY(Gemv, RuntimeType::RT_CUDA, uint8_t, ImplType::CUDA));
  MACE_REGISTER_DELEGATOR(registry, cuda::q8::Conv2d, delegator::Conv2dParam,
                          MACE_DELEGATOR_KEY(Conv2d, RuntimeType::RT_CUDA, uint8_t, ImplType::CUDA));
  MACE_REGISTER_DELEGATOR(
      registry, cuda::q8::DepthwiseConv2d, delegator::DepthwiseConv2dParam,
      MACE_DELEGATOR_KEY(DepthwiseConv2d, RuntimeType::RT_CUDA, uint8_t, ImplType::CUDA));
  MACE_REGISTER_DELEGATOR(registry, cuda::fp32::Gemm, delegator::GemmParam,
                          MACE_DELEGATOR_KEY(Gemm, RuntimeType::RT_CUDA, float, ImplType::CUDA));
  MACE_REGISTER_DELEGATOR(registry, cuda::fp32::Gemv, DelegatorParam,
                          MACE_DELEGATOR_KEY(Gemv, RuntimeType::RT_CUDA, float, ImplType::CUDA));
  MACE_REGISTER_DELEGATOR(registry, cuda::fp32::Conv2d, delegator::Conv2dParam,
                          MACE_DELEGATOR_KEY(Conv2d, RuntimeType::RT_CUDA, float, ImplType::CUDA));
  MACE_REGISTER_DELEGATOR(
      registry, cuda::fp32::Conv2d, delegator::Conv2dParam,
      MACE_DELEGATOR_KEY_EX(Conv2d, RuntimeType::RT_CUDA, float, ImplType::CUDA, K1x1));
  MACE_REGISTER_DELEGATOR(
      registry, cuda::fp32::Conv2dK3x3Winograd, delegator::Conv2dParam,
      MACE_DELEGATOR_KEY_EX(Conv2d, RuntimeType::RT_CUDA, float, ImplType::CUDA, K3x3Winograd));
  MACE_REGISTER_DELEGATOR(
      registry, cuda::fp32::DepthwiseConv2d, delegator::DepthwiseConv2dParam,
      MACE_DELEGATOR_KEY(DepthwiseConv2d, RuntimeType::RT_CUDA, float, ImplType::CUDA));
}

}  // namespace ops
}  // namespace mace
