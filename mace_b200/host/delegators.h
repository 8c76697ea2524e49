// Abstract kernel interfaces of the hot path, with the signatures of MACE's
// delegator headers:
//   delegator::Gemm / GemmParam      mace/ops/delegator/gemm.h:28-70
//   delegator::Gemv                  mace/ops/delegator/gemv.h:27-45
//   delegator::Conv2d / Conv2dParam  mace/ops/delegator/conv_2d.h:46-82
//   delegator::DepthwiseConv2d       mace/ops/delegator/depthwise_conv_2d.h:25-26
// and the registration entry point for the CUDA implementations (the analogue
// of RegisterAllOpDelegators, mace/ops/registry/op_delegators_registry.cc:87-143).
#ifndef MACE_B200_HOST_DELEGATORS_H_
#define MACE_B200_HOST_DELEGATORS_H_

#include <vector>

#include "core.h"
#include "quantize_util.h"

namespace mace {
namespace ops {

enum ConvType {  // mace/ops/delegator/conv_2d.h:28-41, the same values
  K1x1,
  K1x7S1,
  K7x1S1,
  K1x15S1,
  K15x1S1,
  K3x3S1,
  K3x3S2,
  K3x3Winograd,
  K5x5S1,
  K7x7S1,
  K7x7S2,
  K7x7S3,
};

enum ActivationType {  // mace/ops/common/activation_type.h:21-31
  NOOP = 0, RELU = 1, RELUX = 2, PRELU = 3, TANH = 4, SIGMOID = 5, LEAKYRELU = 6, ELU = 7,
  HARDSIGMOID = 8,
};

namespace delegator {

struct GemmParam : public DelegatorParam {
  explicit GemmParam(const bool should_cache_pack = false) : should_cache_pack_(should_cache_pack) {}
  const bool should_cache_pack_;
};

class Gemm : public OpDelegator {
 public:
  explicit Gemm(const GemmParam &param) : OpDelegator(param) {}
  virtual ~Gemm() = default;
  MACE_DEFINE_DELEGATOR_CREATOR(Gemm)

  virtual MaceStatus Compute(const OpContext *context, const Tensor *lhs, const Tensor *rhs,
                             const index_t batch, const index_t rows, const index_t cols,
                             const index_t depth, const MatrixMajor lhs_major,
                             const MatrixMajor rhs_major, const MatrixMajor output_major,
                             const bool lhs_batched, const bool rhs_batched, Tensor *output) = 0;
  // Original matrices are row-major before the transposes.
  virtual MaceStatus Compute(const OpContext *context, const Tensor *lhs, const Tensor *rhs,
                             const index_t batch, const index_t lhs_rows, const index_t lhs_cols,
                             const index_t rhs_rows, const index_t rhs_cols,
                             const bool transpose_lhs, const bool transpose_rhs,
                             const bool transpose_out, const bool lhs_batched,
                             const bool rhs_batched, Tensor *output) = 0;
};

class Gemv : public OpDelegator {
 public:
  explicit Gemv(const DelegatorParam &param) : OpDelegator(param) {}
  virtual ~Gemv() = default;
  MACE_DEFINE_DELEGATOR_CREATOR(Gemv)

  // Always row-major after transpose.
  virtual MaceStatus Compute(const OpContext *context, const Tensor *lhs, const Tensor *rhs,
                             const Tensor *bias, const index_t batch, const index_t lhs_height,
                             const index_t lhs_width, const bool lhs_batched,
                             const bool rhs_batched, Tensor *output) = 0;
};

struct Conv2dParam : public DelegatorParam {
  explicit Conv2dParam(const std::vector<int> &strides, const std::vector<int> &dilations,
                       const std::vector<int> &paddings, const Padding padding_type)
      : strides_(strides), dilations_(dilations), paddings_(paddings), padding_type_(padding_type) {}
  const std::vector<int> &strides_;
  const std::vector<int> &dilations_;
  const std::vector<int> &paddings_;
  const Padding padding_type_;
};

class Conv2d : public OpDelegator {
 public:
  explicit Conv2d(const Conv2dParam &param)
      : OpDelegator(param), strides_(param.strides_), dilations_(param.dilations_),
        paddings_(param.paddings_), padding_type_(param.padding_type_) {}
  virtual ~Conv2d() = default;
  MACE_DEFINE_DELEGATOR_CREATOR(Conv2d)

  virtual MaceStatus Compute(const OpContext *context, const Tensor *input, const Tensor *filter,
                             Tensor *output) = 0;
  // The quantized kernels fuse the int32 bias into the GEMM epilogue (the CPU
  // op passes it to the gemmlowp pipeline, mace/ops/conv_2d.cc:308-310); the
  // op hands it over before Compute.  The fp32 kernels also fuse the bias add
  // and the activation that the CPU op runs as two more passes
  // (mace/ops/conv_2d.cc:171-173).
  void SetBias(const Tensor *bias) { bias_ = bias; }
  void SetActivation(int type, float max_limit, float coefficient) {
    activation_ = type;
    max_limit_ = max_limit;
    coefficient_ = coefficient;
  }
  // A tensor shaped like the output that is added before the activation (a residual sum merged
  // into the convolution by the net); delegators that cannot fuse it ignore the setter's
  // return value at their peril, so it says whether the delegator will apply it.
  virtual bool SetResidual(const Tensor *residual) {
    (void)residual;
    return false;
  }

 protected:
  const std::vector<int> strides_;
  const std::vector<int> dilations_;
  const std::vector<int> paddings_;
  const Padding padding_type_;
  const Tensor *bias_ = nullptr;
  int activation_ = 0;  // ops::ActivationType value
  float max_limit_ = 0.f, coefficient_ = 0.f;
};

typedef Conv2d DepthwiseConv2d;
typedef Conv2dParam DepthwiseConv2dParam;

}  // namespace delegator

// Registers the CUDA delegators of this library:
//   (Gemm, RT_CUDA, uint8_t, CUDA), (Gemv, RT_CUDA, uint8_t, CUDA),
//   (Conv2d, RT_CUDA, uint8_t, CUDA, general), (DepthwiseConv2d, RT_CUDA, uint8_t, CUDA)
//   (Gemm | Gemv | DepthwiseConv2d, RT_CUDA, float, CUDA),
//   (Conv2d, RT_CUDA, float, CUDA, general | K1x1 | K3x3Winograd)
void RegisterAllCudaOpDelegators(OpDelegatorRegistry *registry);

}  // namespace ops
}  // namespace mace

#endif  // MACE_B200_HOST_DELEGATORS_H_
