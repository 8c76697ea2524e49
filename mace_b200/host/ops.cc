#include "ops.h"

#include <sstream>

#include "logging.h"

#include <algorithm>
#include <numeric>
#include <set>
#include <type_traits>

namespace mace {

// ---- Operation ---------------------------------------------------------------

Operation::Operation(OpConstructContext *context) : operator_def_(context->operator_def()) {}

template <>
int Operation::GetOptionalArg<int>(const std::string &name, const int &default_value) const {
  auto it = operator_def_->i.find(name);
  return it == operator_def_->i.end() ? default_value : it->second;
}

template <>
bool Operation::GetOptionalArg<bool>(const std::string &name, const bool &default_value) const {
  auto it = operator_def_->i.find(name);
  return it == operator_def_->i.end() ? default_value : it->second != 0;
}

template <>
float Operation::GetOptionalArg<float>(const std::string &name, const float &default_value) const {
  auto it = operator_def_->f.find(name);
  return it == operator_def_->f.end() ? default_value : it->second;
}

template <>
std::string Operation::GetOptionalArg<std::string>(const std::string &name,
                                                   const std::string &default_value) const {
  auto it = operator_def_->s.find(name);
  return it == operator_def_->s.end() ? default_value : it->second;
}

template <>
std::vector<int> Operation::GetRepeatedArgs<int>(const std::string &name,
                                                 const std::vector<int> &default_value) const {
  auto it = operator_def_->ints.find(name);
  return it == operator_def_->ints.end() ? default_value : it->second;
}

template <>
std::vector<float> Operation::GetRepeatedArgs<float>(const std::string &name,
                                                     const std::vector<float> &default_value) const {
  auto it = operator_def_->floats.find(name);
  return it == operator_def_->floats.end() ? default_value : it->second;
}

MaceStatus Operation::Init(OpConstructContext *context) {
  Workspace *ws = context->workspace();
  for (const std::string &name : operator_def_->input) {
    const Tensor *t = ws->GetTensor(name);
    if (t == nullptr)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS,
                        "op " + operator_def_->name + ": Input does not exist in workspace: " + name);
    inputs_.push_back(t);
  }
  for (size_t i = 0; i < operator_def_->output.size(); ++i) {
    const std::string &name = operator_def_->output[i];
    Tensor *t = ws->GetTensor(name);
    if (t == nullptr) {
      DataType dt = static_cast<DataType>(GetOptionalArg<int>("T", static_cast<int>(DT_FLOAT)));
      if (i < operator_def_->output_type.size()) dt = operator_def_->output_type[i];
      t = ws->CreateTensor(name, context->runtime(), dt);
    }
    // mace/core/workspace.cc:204-222: activation ranges come from quantize_info
    if (i < operator_def_->quantize_info.size()) {
      t->SetScale(operator_def_->quantize_info[i].scale);
      t->SetZeroPoint(operator_def_->quantize_info[i].zero_point);
    }
    outputs_.push_back(t);
  }
  return MaceStatus::MACE_SUCCESS;
}

// ---- registry ------------------------------------------------------------------

static std::string OpKey(const std::string &type, RuntimeType rt, DataType dt) {
  return type + "_" + std::to_string(static_cast<int>(rt)) + "_" + std::to_string(static_cast<int>(dt));
}

MaceStatus OpRegistry::Register(const std::string &type, RuntimeType rt, DataType dt, OpCreator creator) {
  registry_[OpKey(type, rt, dt)] = std::move(creator);
  return MaceStatus::MACE_SUCCESS;
}

std::unique_ptr<Operation> OpRegistry::CreateOperation(OpConstructContext *context, RuntimeType rt,
                                                       DataType dt, MaceStatus *status) const {
  auto it = registry_.find(OpKey(context->operator_def()->type, rt, dt));
  if (it == registry_.end()) {
    *status = MaceStatus(MaceStatus::MACE_UNSUPPORTED,
                         "no operator registered for " + context->operator_def()->type);
    return nullptr;
  }
  *status = MaceStatus::MACE_SUCCESS;
  return it->second(context);
}

namespace ops {

// ---- ConvPool2dOpBase (mace/ops/conv_pool_2d_base.h:25-46) -------------------------

class ConvPool2dOpBase : public Operation {
 public:
  explicit ConvPool2dOpBase(OpConstructContext *context)
      : Operation(context),
        strides_(GetRepeatedArgs<int>("strides")),
        padding_type_(static_cast<Padding>(GetOptionalArg<int>("padding", static_cast<int>(SAME)))),
        paddings_(GetRepeatedArgs<int>("padding_values")),
        dilations_(GetRepeatedArgs<int>("dilations", {1, 1})) {}

 protected:
  std::vector<int> strides_;
  Padding padding_type_;
  std::vector<int> paddings_;
  std::vector<int> dilations_;
};

template <RuntimeType D, class T> class Conv2dOp;
template <RuntimeType D, class T> class DepthwiseConv2dOp;
template <RuntimeType D, class T> class MatMulOp;
template <RuntimeType D, class T> class FullyConnectedOp;
template <RuntimeType D, class T> class PoolingOp;
template <RuntimeType D, class T> class EltwiseOp;
template <RuntimeType D, class T> class ActivationOp;
template <RuntimeType D, class T> class SoftmaxOp;
template <RuntimeType D, class T> class QuantizeOp;
template <RuntimeType D, class T> class DequantizeOp;
template <RuntimeType D, class T> class TransposeOp;
template <RuntimeType D, class T> class SqueezeOp;
template <RuntimeType D, class T> class ReshapeOp;
template <RuntimeType D, class T> class SubsampleOp;

template <>
class Conv2dOp<RuntimeType::RT_CUDA, uint8_t> : public ConvPool2dOpBase {
 public:
  explicit Conv2dOp(OpConstructContext *context)
      : ConvPool2dOpBase(context), workspace_(context->workspace()) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0), *filter = Input(1);
    const Tensor *bias = InputSize() >= 3 ? Input(2) : nullptr;
    if (strides_.size() != 2) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "strides must have 2 values");
    if (conv2d_delegator_ == nullptr) {
      // one CUDA implementation serves every filter shape (tag "general")
      conv2d_delegator_ = delegator::Conv2d::Create(
          workspace_, MACE_DELEGATOR_KEY(Conv2d, RuntimeType::RT_CUDA, uint8_t, ImplType::CUDA),
          delegator::Conv2dParam(strides_, dilations_, paddings_, padding_type_));
    }
    MACE_RETURN_IF_NO_DELEGATOR(conv2d_delegator_, workspace_);
    conv2d_delegator_->SetBias(bias);
    return conv2d_delegator_->Compute(context, input, filter, Output(0));
  }

 private:
  Workspace *workspace_;
  std::unique_ptr<delegator::Conv2d> conv2d_delegator_;
};

static ActivationType StringToActivationType(const std::string &type, MaceStatus *status) {
  *status = MaceStatus::MACE_SUCCESS;
  if (type == "NOOP") return NOOP;
  if (type == "RELU") return RELU;
  if (type == "RELUX") return RELUX;
  if (type == "LEAKYRELU") return LEAKYRELU;
  *status = MaceStatus(MaceStatus::MACE_UNSUPPORTED, "activation not fused by the CUDA runtime: " + type);
  return NOOP;
}

// fp32 Conv2D, NCHW: delegator choice as Conv2dOp<RT_CPU,T>::Run makes it on first use
// (mace/ops/conv_2d.cc:88-169): 1x1 stride 1 -> K1x1; 3x3 stride 1 with at least 8 input and 8
// output channels -> K3x3Winograd; everything else -> general.  Bias and activation are
// handed to the delegator, which fuses them.
template <>
class Conv2dOp<RuntimeType::RT_CUDA, float> : public ConvPool2dOpBase {
 public:
  explicit Conv2dOp(OpConstructContext *context)
      : ConvPool2dOpBase(context), workspace_(context->workspace()),
        activation_name_(GetOptionalArg<std::string>("activation", "NOOP")),
        max_limit_(GetOptionalArg<float>("max_limit", 0.0f)),
        coefficient_(GetOptionalArg<float>("activation_coefficient", 0.0f)) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0), *filter = Input(1);
    // (an absorbed residual is appended to the inputs, so that the net sees its last reader)
    const int own_inputs = InputSize() - (residual_ != nullptr ? 1 : 0);
    const Tensor *bias = own_inputs >= 3 ? Input(2) : nullptr;
    if (strides_.size() != 2) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "strides must have 2 values");
    MaceStatus st;
    const ActivationType act = StringToActivationType(activation_name_, &st);
    MACE_RETURN_IF_ERROR(st);
    if (conv2d_delegator_ == nullptr) {
      const index_t filter_h = filter->dim(2), filter_w = filter->dim(3);
      const index_t in_channels = input->dim(1), out_channels = filter->dim(0);
      const bool s1d1 = strides_[0] == 1 && strides_[1] == 1 && dilations_[0] == 1 && dilations_[1] == 1;
      delegator::Conv2dParam param(strides_, dilations_, paddings_, padding_type_);
      if (filter_h == 1 && filter_w == 1 && s1d1) {
        conv2d_delegator_ = delegator::Conv2d::Create(
            workspace_, MACE_DELEGATOR_KEY_EX(Conv2d, RuntimeType::RT_CUDA, float, ImplType::CUDA, K1x1), param);
      } else if (filter_h == 3 && filter_w == 3 && s1d1 && in_channels >= 8 && out_channels >= 8) {
        conv2d_delegator_ = delegator::Conv2d::Create(
            workspace_,
            MACE_DELEGATOR_KEY_EX(Conv2d, RuntimeType::RT_CUDA, float, ImplType::CUDA, K3x3Winograd), param);
      } else {
        conv2d_delegator_ = delegator::Conv2d::Create(
            workspace_, MACE_DELEGATOR_KEY(Conv2d, RuntimeType::RT_CUDA, float, ImplType::CUDA), param);
      }
    }
    MACE_RETURN_IF_NO_DELEGATOR(conv2d_delegator_, workspace_);
    conv2d_delegator_->SetBias(bias);
    if (residual_ != nullptr) {
      conv2d_delegator_->SetActivation(sum_.activation, sum_.max_limit, sum_.coefficient);
    } else {
      conv2d_delegator_->SetActivation(act, max_limit_, coefficient_);
    }
    return conv2d_delegator_->Compute(context, input, filter, Output(0));
  }

  bool DescribeStridedPointwise(int *stride_h, int *stride_w) const override {
    const Tensor *filter = Input(1);
    if (residual_ != nullptr || strides_.size() != 2 || filter->dim_size() != 4) return false;
    if (filter->dim(2) != 1 || filter->dim(3) != 1 || (strides_[0] == 1 && strides_[1] == 1)) return false;
    if (strides_[0] < 1 || strides_[1] < 1 || dilations_.size() != 2 || dilations_[0] != 1 || dilations_[1] != 1)
      return false;
    // SAME and VALID both pad a 1x1 filter by nothing; explicit padding values must be zero
    for (int pad : paddings_)
      if (pad != 0) return false;
    if (paddings_.empty() && padding_type_ != SAME && padding_type_ != VALID) return false;
    *stride_h = strides_[0];
    *stride_w = strides_[1];
    return true;
  }

  void TakeSubsampledInput(const Tensor *subsampled) override {
    inputs_[0] = subsampled;
    strides_ = {1, 1};
    conv2d_delegator_.reset();  // the next Run() picks the 1x1 delegator
  }

  // Needs the delegator, i.e. one Run() before the net merges operators.
  bool AbsorbResidualSum(const Tensor *residual, const ResidualSum &sum, Tensor *sum_output) override {
    if (residual_ != nullptr || conv2d_delegator_ == nullptr || activation_name_ != "NOOP") return false;
    if (!conv2d_delegator_->SetResidual(residual)) return false;
    residual_ = residual;
    sum_ = sum;
    inputs_.push_back(residual);
    outputs_[0] = sum_output;
    return true;
  }

 private:
  Workspace *workspace_;
  std::string activation_name_;
  float max_limit_, coefficient_;
  std::unique_ptr<delegator::Conv2d> conv2d_delegator_;
  const Tensor *residual_ = nullptr;
  ResidualSum sum_;
};

template <>
class DepthwiseConv2dOp<RuntimeType::RT_CUDA, float> : public ConvPool2dOpBase {
 public:
  explicit DepthwiseConv2dOp(OpConstructContext *context)
      : ConvPool2dOpBase(context), workspace_(context->workspace()),
        activation_name_(GetOptionalArg<std::string>("activation", "NOOP")),
        max_limit_(GetOptionalArg<float>("max_limit", 0.0f)),
        coefficient_(GetOptionalArg<float>("activation_coefficient", 0.0f)) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0), *filter = Input(1);
    const Tensor *bias = InputSize() >= 3 ? Input(2) : nullptr;
    if (strides_.size() != 2) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "strides must have 2 values");
    MaceStatus st;
    const ActivationType act = StringToActivationType(activation_name_, &st);
    MACE_RETURN_IF_ERROR(st);
    if (delegator_ == nullptr) {
      delegator_ = delegator::DepthwiseConv2d::Create(
          workspace_, MACE_DELEGATOR_KEY(DepthwiseConv2d, RuntimeType::RT_CUDA, float, ImplType::CUDA),
          delegator::DepthwiseConv2dParam(strides_, dilations_, paddings_, padding_type_));
    }
    MACE_RETURN_IF_NO_DELEGATOR(delegator_, workspace_);
    delegator_->SetBias(bias);
    delegator_->SetActivation(act, max_limit_, coefficient_);
    return delegator_->Compute(context, input, filter, Output(0));
  }

 private:
  Workspace *workspace_;
  std::string activation_name_;
  float max_limit_, coefficient_;
  std::unique_ptr<delegator::DepthwiseConv2d> delegator_;
};

// fp32 MatMul (mace/ops/matmul.cc:96-225): batched GEMM through the Gemm delegator; a bias
// input is not supported by this runtime (MACE_UNSUPPORTED).
template <>
class MatMulOp<RuntimeType::RT_CUDA, float> : public Operation {
 public:
  explicit MatMulOp(OpConstructContext *context)
      : Operation(context), registry_workspace_(context->workspace()),
        transpose_a_(GetOptionalArg<bool>("transpose_a", false)),
        transpose_b_(GetOptionalArg<bool>("transpose_b", false)),
        gemm_(delegator::Gemm::Create(context->workspace(),
                                      MACE_DELEGATOR_KEY(Gemm, RuntimeType::RT_CUDA, float, ImplType::CUDA),
                                      delegator::GemmParam())) {}

  MaceStatus Run(OpContext *context) override {
    MACE_RETURN_IF_NO_DELEGATOR(gemm_, registry_workspace_);
    const Tensor *lhs = Input(0), *rhs = Input(1);
    if (InputSize() >= 3) return MaceStatus(MaceStatus::MACE_UNSUPPORTED, "MatMul bias input");
    Tensor *C = Output(0);
    const index_t lhs_rank = lhs->dim_size(), rhs_rank = rhs->dim_size();
    if (lhs_rank < 2 || rhs_rank < 2)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "rank should be greater than or equal to 2");
    if (lhs_rank == rhs_rank) {
      for (index_t i = 0; i < lhs_rank - 2; ++i)
        if (lhs->dim(i) != rhs->dim(i))
          return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "batch dimensions are not equal");
    } else if (lhs_rank != 2 && rhs_rank != 2) {
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS,
                        "Either lhs or rhs matrix should has rank 2 for non-batched matrix multiplication");
    }
    const index_t lhs_rows = lhs->dim(lhs_rank - 2), lhs_cols = lhs->dim(lhs_rank - 1);
    const index_t rhs_rows = rhs->dim(rhs_rank - 2), rhs_cols = rhs->dim(rhs_rank - 1);
    const index_t rows = transpose_a_ ? lhs_cols : lhs_rows;
    const index_t cols = transpose_b_ ? rhs_rows : rhs_cols;
    const index_t depth = transpose_a_ ? lhs_rows : lhs_cols;
    if (depth != (transpose_b_ ? rhs_cols : rhs_rows))
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "the number of A's column must be equal to B's row");
    const index_t lhs_batch = std::accumulate(lhs->shape().begin(), lhs->shape().end() - 2,
                                              static_cast<index_t>(1), std::multiplies<index_t>());
    const index_t rhs_batch = std::accumulate(rhs->shape().begin(), rhs->shape().end() - 2,
                                              static_cast<index_t>(1), std::multiplies<index_t>());
    std::vector<index_t> output_shape = lhs_rank >= rhs_rank ? lhs->shape() : rhs->shape();
    output_shape[output_shape.size() - 2] = rows;
    output_shape[output_shape.size() - 1] = cols;
    const index_t batch = lhs_rank >= rhs_rank ? lhs_batch : rhs_batch;
    MACE_RETURN_IF_ERROR(C->Resize(output_shape));
    return gemm_->Compute(context, lhs, rhs, batch, rows, cols, depth,
                          transpose_a_ ? ColMajor : RowMajor, transpose_b_ ? ColMajor : RowMajor,
                          RowMajor, !(lhs_rank < rhs_rank), !(rhs_rank < lhs_rank), C);
  }

 private:
  Workspace *registry_workspace_;
  bool transpose_a_, transpose_b_;
  std::unique_ptr<delegator::Gemm> gemm_;
};

// fp32 FullyConnected (mace/ops/fully_connected.cc:61-125): weight OIHW, input NCHW, output
// [N, O, 1, 1]; Gemv with the weight as the matrix.  Only NOOP activation is supported here.
template <>
class FullyConnectedOp<RuntimeType::RT_CUDA, float> : public Operation {
 public:
  explicit FullyConnectedOp(OpConstructContext *context)
      : Operation(context), registry_workspace_(context->workspace()),
        activation_name_(GetOptionalArg<std::string>("activation", "NOOP")),
        gemv_(delegator::Gemv::Create(context->workspace(),
                                      MACE_DELEGATOR_KEY(Gemv, RuntimeType::RT_CUDA, float, ImplType::CUDA),
                                      DelegatorParam())) {}

  MaceStatus Run(OpContext *context) override {
    MACE_RETURN_IF_NO_DELEGATOR(gemv_, registry_workspace_);
    const Tensor *input = Input(0), *weight = Input(1);
    const Tensor *bias = InputSize() >= 3 ? Input(2) : nullptr;
    Tensor *output = Output(0);
    if (activation_name_ != "NOOP")
      return MaceStatus(MaceStatus::MACE_UNSUPPORTED, "FullyConnected activation " + activation_name_);
    if (!(input->dim(1) == weight->dim(1) && input->dim(2) == weight->dim(2) &&
          input->dim(3) == weight->dim(3)))
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "The shape of Input and Weight don't match.");
    if (bias != nullptr && weight->dim(0) != bias->dim(0))
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "The shape of Weight and Bias don't match.");
    MACE_RETURN_IF_ERROR(output->Resize({input->dim(0), weight->dim(0), 1, 1}));
    return gemv_->Compute(context, weight, input, bias, output->dim(0), weight->dim(0),
                          weight->dim(1) * weight->dim(2) * weight->dim(3), false, true, output);
  }

 private:
  Workspace *registry_workspace_;
  std::string activation_name_;
  std::unique_ptr<delegator::Gemv> gemv_;
};

template <>
class DepthwiseConv2dOp<RuntimeType::RT_CUDA, uint8_t> : public ConvPool2dOpBase {
 public:
  explicit DepthwiseConv2dOp(OpConstructContext *context)
      : ConvPool2dOpBase(context), workspace_(context->workspace()) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0), *filter = Input(1);
    const Tensor *bias = InputSize() >= 3 ? Input(2) : nullptr;
    if (strides_.size() != 2) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "strides must have 2 values");
    if (delegator_ == nullptr) {
      delegator_ = delegator::DepthwiseConv2d::Create(
          workspace_, MACE_DELEGATOR_KEY(DepthwiseConv2d, RuntimeType::RT_CUDA, uint8_t, ImplType::CUDA),
          delegator::DepthwiseConv2dParam(strides_, dilations_, paddings_, padding_type_));
    }
    MACE_RETURN_IF_NO_DELEGATOR(delegator_, workspace_);
    delegator_->SetBias(bias);
    return delegator_->Compute(context, input, filter, Output(0));
  }

 private:
  Workspace *workspace_;
  std::unique_ptr<delegator::DepthwiseConv2d> delegator_;
};

template <>
class MatMulOp<RuntimeType::RT_CUDA, uint8_t> : public Operation {
 public:
  explicit MatMulOp(OpConstructContext *context)
      : Operation(context), registry_workspace_(context->workspace()),
        transpose_a_(GetOptionalArg<bool>("transpose_a", false)),
        transpose_b_(GetOptionalArg<bool>("transpose_b", false)),
        gemm_(delegator::Gemm::Create(
            context->workspace(),
            MACE_DELEGATOR_KEY(Gemm, RuntimeType::RT_CUDA, uint8_t, ImplType::CUDA),
            delegator::GemmParam())) {}

  MaceStatus Run(OpContext *context) override {
    MACE_RETURN_IF_NO_DELEGATOR(gemm_, registry_workspace_);
    const Tensor *lhs = Input(0), *rhs = Input(1);
    Tensor *C = Output(0);
    const index_t lhs_rank = lhs->dim_size(), rhs_rank = rhs->dim_size();
    // Validate(), mace/ops/matmul.cc:55-83
    if (lhs_rank < 2 || rhs_rank < 2)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "rank should be greater than or equal to 2");
    if (lhs_rank == rhs_rank) {
      for (index_t i = 0; i < lhs_rank - 2; ++i)
        if (lhs->dim(i) != rhs->dim(i))
          return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "batch dimensions are not equal");
    } else if (lhs_rank != 2 && rhs_rank != 2) {
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS,
                        "Either lhs or rhs matrix should has rank 2 for non-batched matrix multiplication");
    }
    const index_t lhs_rows = lhs->dim(lhs_rank - 2), lhs_cols = lhs->dim(lhs_rank - 1);
    const index_t rhs_rows = rhs->dim(rhs_rank - 2), rhs_cols = rhs->dim(rhs_rank - 1);
    const index_t rows = transpose_a_ ? lhs_cols : lhs_rows;
    const index_t cols = transpose_b_ ? rhs_rows : rhs_cols;
    const index_t depth = transpose_a_ ? lhs_rows : lhs_cols;
    const index_t rhs_depth = transpose_b_ ? rhs_cols : rhs_rows;
    if (depth != rhs_depth)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "the number of A's column must be equal to B's row");
    const index_t lhs_batch = std::accumulate(lhs->shape().begin(), lhs->shape().end() - 2,
                                              static_cast<index_t>(1), std::multiplies<index_t>());
    const index_t rhs_batch = std::accumulate(rhs->shape().begin(), rhs->shape().end() - 2,
                                              static_cast<index_t>(1), std::multiplies<index_t>());
    std::vector<index_t> output_shape;
    index_t batch = 1;
    if (lhs_rank >= rhs_rank) {
      output_shape = lhs->shape();
      output_shape[lhs_rank - 2] = rows;
      output_shape[lhs_rank - 1] = cols;
      batch = lhs_batch;
    } else {
      output_shape = rhs->shape();
      output_shape[rhs_rank - 2] = rows;
      output_shape[rhs_rank - 1] = cols;
      batch = rhs_batch;
    }
    const bool lhs_batched = !(lhs_rank < rhs_rank), rhs_batched = !(rhs_rank < lhs_rank);
    MACE_RETURN_IF_ERROR(C->Resize(output_shape));
    // The quantized MatMul reads no bias input (MakeNoBias, matmul.cc:280).
    return gemm_->Compute(context, lhs, rhs, batch, rows, cols, depth,
                          transpose_a_ ? ColMajor : RowMajor, transpose_b_ ? ColMajor : RowMajor,
                          RowMajor, lhs_batched, rhs_batched, C);
  }

 private:
  Workspace *registry_workspace_;
  bool transpose_a_, transpose_b_;
  std::unique_ptr<delegator::Gemm> gemm_;
};

template <>
class FullyConnectedOp<RuntimeType::RT_CUDA, uint8_t> : public Operation {
 public:
  explicit FullyConnectedOp(OpConstructContext *context)
      : Operation(context), registry_workspace_(context->workspace()),
        gemv_(delegator::Gemv::Create(
            context->workspace(),
            MACE_DELEGATOR_KEY(Gemv, RuntimeType::RT_CUDA, uint8_t, ImplType::CUDA),
            DelegatorParam())) {}

  MaceStatus Run(OpContext *context) override {
    MACE_RETURN_IF_NO_DELEGATOR(gemv_, registry_workspace_);
    const Tensor *input = Input(0), *weight = Input(1);
    const Tensor *bias = InputSize() >= 3 ? Input(2) : nullptr;
    Tensor *output = Output(0);
    if (!(input->dim(1) == weight->dim(1) && input->dim(2) == weight->dim(2) &&
          input->dim(3) == weight->dim(3)))
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "The shape of Input and Weight don't match.");
    if (bias != nullptr && weight->dim(0) != bias->dim(0))
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "The shape of Weight and Bias don't match.");
    MACE_RETURN_IF_ERROR(output->Resize({input->dim(0), 1, 1, weight->dim(0)}));
    const index_t input_size = weight->dim(1) * weight->dim(2) * weight->dim(3);
    return gemv_->Compute(context, weight, input, bias, output->dim(0), weight->dim(0), input_size,
                          false, true, output);
  }

 private:
  Workspace *registry_workspace_;
  std::unique_ptr<delegator::Gemv> gemv_;
};

template <>
class PoolingOp<RuntimeType::RT_CUDA, uint8_t> : public ConvPool2dOpBase {
 public:
  explicit PoolingOp(OpConstructContext *context)
      : ConvPool2dOpBase(context),
        kernels_(GetRepeatedArgs<int>("kernels")),
        pooling_type_(static_cast<PoolingType>(GetOptionalArg<int>("pooling_type", static_cast<int>(AVG)))),
        round_type_(static_cast<RoundType>(GetOptionalArg<int>("round_mode", static_cast<int>(CEIL)))) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0);
    Tensor *output = Output(0);
    if (dilations_[0] != 1 || dilations_[1] != 1)
      return MaceStatus(MaceStatus::MACE_UNSUPPORTED, "Quantized pooling does not support dilation > 1 yet.");
    if (pooling_type_ != AVG)
      return MaceStatus(MaceStatus::MACE_UNSUPPORTED, "only AVG pooling is built for the CUDA runtime");
    if (kernels_.size() != 2 || strides_.size() != 2)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "kernels and strides must have 2 values");
    // Use the same scale and zero point with input and output (pooling.cc:651-653).
    output->SetScale(input->scale());
    output->SetZeroPoint(input->zero_point());
    index_t out_h = 0, out_w = 0;
    std::vector<int> paddings(2);
    if (paddings_.empty()) {
      MACE_RETURN_IF_ERROR(CalcPaddingAndOutputSize(input->dim(1), input->dim(2), kernels_[0], kernels_[1],
                                                    dilations_.data(), strides_.data(), padding_type_,
                                                    &out_h, &out_w, paddings.data()));
    } else {
      paddings = paddings_;
      CalcOutputSize(input->dim(1), input->dim(2), kernels_[0], kernels_[1], paddings.data(),
                     dilations_.data(), strides_.data(), round_type_, &out_h, &out_w);
    }
    MACE_RETURN_IF_ERROR(output->Resize({input->dim(0), out_h, out_w, input->dim(3)}));
    CudaRuntime *rt = CudaRuntimeOf(context);
    return rt->Status(mb_avgpool_u8_nhwc(rt->ctx(), input->memory<uint8_t>(),
                                         output->mutable_memory<uint8_t>(), input->dim(0), input->dim(1),
                                         input->dim(2), input->dim(3), kernels_[0], kernels_[1],
                                         strides_[0], strides_[1], paddings[0] / 2, paddings[1] / 2,
                                         out_h, out_w));
  }

 private:
  std::vector<int> kernels_;
  PoolingType pooling_type_;
  RoundType round_type_;
};

// fp32 Pooling, NCHW (mace/ops/pooling.cc:46-126): MAX and AVG, output size from the padding
// type or from explicit paddings with round_mode (CEIL unless the arg says FLOOR).
template <>
class PoolingOp<RuntimeType::RT_CUDA, float> : public ConvPool2dOpBase {
 public:
  explicit PoolingOp(OpConstructContext *context)
      : ConvPool2dOpBase(context),
        kernels_(GetRepeatedArgs<int>("kernels")),
        pooling_type_(static_cast<PoolingType>(GetOptionalArg<int>("pooling_type", static_cast<int>(AVG)))),
        round_type_(static_cast<RoundType>(GetOptionalArg<int>("round_mode", static_cast<int>(CEIL)))) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0);
    Tensor *output = Output(0);
    if (input->dim_size() != 4) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Pooling input must be NCHW");
    if (kernels_.size() != 2 || strides_.size() != 2)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "kernels and strides must have 2 values");
    if (pooling_type_ != AVG && pooling_type_ != MAX)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "unknown pooling type");
    index_t out_h = 0, out_w = 0;
    std::vector<int> paddings(2);
    if (paddings_.empty()) {
      MACE_RETURN_IF_ERROR(CalcPaddingAndOutputSize(input->dim(2), input->dim(3), kernels_[0], kernels_[1],
                                                    dilations_.data(), strides_.data(), padding_type_,
                                                    &out_h, &out_w, paddings.data()));
    } else {
      paddings = paddings_;
      CalcOutputSize(input->dim(2), input->dim(3), kernels_[0], kernels_[1], paddings.data(),
                     dilations_.data(), strides_.data(), round_type_, &out_h, &out_w);
    }
    MACE_RETURN_IF_ERROR(output->Resize({input->dim(0), input->dim(1), out_h, out_w}));
    CudaRuntime *rt = CudaRuntimeOf(context);
    // pad_hw = paddings / 2 (pooling.cc:104-105)
    return rt->Status(mb_pooling_f32_nchw(rt->ctx(), input->memory<float>(), output->mutable_memory<float>(),
                                          input->dim(0), input->dim(1), input->dim(2), input->dim(3),
                                          kernels_[0], kernels_[1], strides_[0], strides_[1], dilations_[0],
                                          dilations_[1], paddings[0] / 2, paddings[1] / 2, out_h, out_w,
                                          static_cast<int>(pooling_type_)));
  }

 private:
  std::vector<int> kernels_;
  PoolingType pooling_type_;
  RoundType round_type_;
};

// fp32 Eltwise (mace/ops/eltwise.cc:949-1144) for the two forms a float network's residual
// adds and scalings use: two inputs of the same size, or one input and the scalar_input arg.
// Broadcasting between different shapes returns MACE_UNSUPPORTED.
template <>
class EltwiseOp<RuntimeType::RT_CUDA, float> : public Operation {
 public:
  explicit EltwiseOp(OpConstructContext *context)
      : Operation(context),
        type_(GetOptionalArg<int>("type", 14 /* NONE */)),
        coeff_(GetRepeatedArgs<float>("coeff")),
        scalar_input_(GetOptionalArg<float>("scalar_input", 1.0f)),
        scalar_input_index_(GetOptionalArg<int>("scalar_input_index", 1)) {}

  MaceStatus Run(OpContext *context) override {
    if (InputSize() >= 3)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Element-Wise does not support 3 or higher inputs");
    const Tensor *input0 = Input(0);
    const Tensor *input1 = InputSize() == 2 ? Input(1) : nullptr;
    if (type_ == 12 /* CLIP */ && !(coeff_.size() == 2 && coeff_[0] < coeff_[1]))
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Clip's min/max values are not correct.");
    if (!coeff_.empty() && coeff_.size() != 2)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "coeff must have 2 values");
    bool swapped = false;
    if (input1 != nullptr) {
      // the larger operand leads (eltwise.cc:1004-1010)
      if (input0->dim_size() < input1->dim_size() ||
          (input0->dim_size() == input1->dim_size() && input0->size() < input1->size())) {
        std::swap(input0, input1);
        swapped = true;
      }
      if (input0->size() != input1->size())
        return MaceStatus(MaceStatus::MACE_UNSUPPORTED, "Eltwise broadcasting is not built for the CUDA runtime");
    }
    if (scalar_input_index_ == 0) swapped = !swapped;
    Tensor *output = Output(0);
    MACE_RETURN_IF_ERROR(output->Resize(input0->shape()));
    CudaRuntime *rt = CudaRuntimeOf(context);
    return rt->Status(mb_eltwise_act_f32(rt->ctx(), input0->memory<float>(),
                                         input1 != nullptr ? input1->memory<float>() : nullptr,
                                         output->mutable_memory<float>(), input0->size(), type_, scalar_input_,
                                         coeff_.empty() ? 0 : 1, coeff_.empty() ? 0.f : coeff_[0],
                                         coeff_.empty() ? 0.f : coeff_[1], swapped ? 1 : 0,
                                         static_cast<int>(fused_act_), fused_max_limit_, fused_coefficient_));
  }

  bool DescribeResidualSum(ResidualSum *sum) const override {
    if (type_ != 0 /* SUM */ || !coeff_.empty() || InputSize() != 2) return false;
    if (Input(0)->size() != Input(1)->size()) return false;
    sum->activation = static_cast<int>(fused_act_);
    sum->max_limit = fused_max_limit_;
    sum->coefficient = fused_coefficient_;
    return true;
  }

  bool AbsorbActivation(const OperatorDef &def, Tensor *activation_output) override {
    if (fused_act_ != NOOP || def.input.size() != 1) return false;  // PRELU has an alpha input
    auto name = def.s.find("activation");
    MaceStatus st;
    const ActivationType act = StringToActivationType(name == def.s.end() ? "NOOP" : name->second, &st);
    if (st != MaceStatus::MACE_SUCCESS) return false;
    auto limit = def.f.find("max_limit"), coef = def.f.find("activation_coefficient");
    fused_act_ = act;
    fused_max_limit_ = limit == def.f.end() ? 0.f : limit->second;
    fused_coefficient_ = coef == def.f.end() ? 0.f : coef->second;
    outputs_[0] = activation_output;
    return true;
  }

 private:
  ActivationType fused_act_ = NOOP;
  float fused_max_limit_ = 0.f, fused_coefficient_ = 0.f;
  int type_;
  std::vector<float> coeff_;
  float scalar_input_;
  int scalar_input_index_;
};

// fp32 Activation (mace/ops/activation.cc:36-79); PRELU (an alpha input) is not built.
template <>
class ActivationOp<RuntimeType::RT_CUDA, float> : public Operation {
 public:
  explicit ActivationOp(OpConstructContext *context)
      : Operation(context),
        activation_name_(GetOptionalArg<std::string>("activation", "NOOP")),
        max_limit_(GetOptionalArg<float>("max_limit", 0.0f)),
        coefficient_(GetOptionalArg<float>("activation_coefficient", 0.0f)) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0);
    Tensor *output = Output(0);
    MaceStatus st;
    const ActivationType act = StringToActivationType(activation_name_, &st);
    MACE_RETURN_IF_ERROR(st);
    MACE_RETURN_IF_ERROR(output->Resize(input->shape()));
    CudaRuntime *rt = CudaRuntimeOf(context);
    return rt->Status(mb_activation_f32(rt->ctx(), input->memory<float>(), output->mutable_memory<float>(),
                                        input->size(), static_cast<int>(act), max_limit_, coefficient_));
  }

 private:
  std::string activation_name_;
  float max_limit_, coefficient_;
};

// fp32 Softmax (mace/ops/softmax.cc:249-290): over the channels of an NCHW tensor when the
// op has a data format and axis 1, otherwise over the last dimension.
template <>
class SoftmaxOp<RuntimeType::RT_CUDA, float> : public Operation {
 public:
  explicit SoftmaxOp(OpConstructContext *context)
      : Operation(context),
        use_log_(GetOptionalArg<bool>("use_log", false)),
        has_df_(GetOptionalArg<int>("has_data_format", 0) != 0),
        axis_(GetOptionalArg<int>("axis", 1)) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0);
    Tensor *output = Output(0);
    if (input->dim_size() < 2) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "The input->dim_size() >= 2 failed.");
    MACE_RETURN_IF_ERROR(output->Resize(input->shape()));
    index_t outer, classes, inner;
    if (input->dim_size() == 4 && has_df_ && axis_ == 1) {
      outer = input->dim(0); classes = input->dim(1); inner = input->dim(2) * input->dim(3);
    } else {
      classes = input->dim(input->dim_size() - 1);
      outer = classes > 0 ? input->size() / classes : 0;
      inner = 1;
    }
    CudaRuntime *rt = CudaRuntimeOf(context);
    return rt->Status(mb_softmax_f32(rt->ctx(), input->memory<float>(), output->mutable_memory<float>(), outer,
                                     classes, inner, use_log_ ? 1 : 0));
  }

 private:
  bool use_log_, has_df_;
  int axis_;
};

// Quantize (mace/ops/quantize.cc:31-74): float -> uint8 with the output tensor's scale and
// zero point, or, when the output has no scale yet (or find_range_every_time), with the
// range of the data; that path reads min and max back to the host and cannot be captured.
template <>
class QuantizeOp<RuntimeType::RT_CUDA, uint8_t> : public Operation {
 public:
  explicit QuantizeOp(OpConstructContext *context)
      : Operation(context),
        non_zero_(GetOptionalArg<int>("non_zero", 0) != 0),
        find_range_every_time_(GetOptionalArg<bool>("find_range_every_time", false)) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0);
    Tensor *output = Output(0);
    if (input->dtype() != DT_FLOAT) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Quantize input must be float");
    MACE_RETURN_IF_ERROR(output->Resize(input->shape()));
    CudaRuntime *rt = CudaRuntimeOf(context);
    if (find_range_every_time_ || !(output->scale() > 0.f)) {
      float mn = 0.f, mx = 0.f, scale = 0.f;
      int32_t zero_point = 0;
      MACE_RETURN_IF_ERROR(rt->Status(mb_minmax_f32(rt->ctx(), input->memory<float>(), input->size(), &mn, &mx)));
      AdjustRangeU8(mn, mx, non_zero_, &scale, &zero_point);
      output->SetScale(scale);
      output->SetZeroPoint(zero_point);
    }
    return rt->Status(mb_quantize_f32_u8(rt->ctx(), input->memory<float>(), output->mutable_memory<uint8_t>(),
                                         input->size(), output->scale(), output->zero_point()));
  }

 private:
  bool non_zero_, find_range_every_time_;
};

// Dequantize (mace/ops/quantize.cc:79-104): uint8 or int32 -> float with the input's scale
// and zero point.
template <class T>
class DequantizeOp<RuntimeType::RT_CUDA, T> : public Operation {
 public:
  explicit DequantizeOp(OpConstructContext *context) : Operation(context) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0);
    Tensor *output = Output(0);
    MACE_RETURN_IF_ERROR(output->Resize(input->shape()));
    CudaRuntime *rt = CudaRuntimeOf(context);
    return rt->Status(mb_dequantize_f32(rt->ctx(), input->memory<T>(), std::is_same<T, int32_t>::value ? 1 : 0,
                                        output->mutable_memory<float>(), input->size(), input->scale(),
                                        input->zero_point()));
  }
};

// Transpose (mace/ops/transpose.cc:34-73) for the permutations that move one block of
// adjacent axes behind the axes that follow it: {0,3,1,2}, {0,2,3,1}, {1,0}, {0,2,1}, ... --
// each a batched 2-D transpose.  Other permutations return MACE_UNSUPPORTED.
template <RuntimeType D, class T>
class TransposeOp : public Operation {
 public:
  explicit TransposeOp(OpConstructContext *context) : Operation(context), dims_(GetRepeatedArgs<int>("dims")) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0);
    Tensor *output = Output(0);
    const std::vector<index_t> &in_shape = input->shape();
    const size_t rank = in_shape.size();
    if (dims_.size() != rank || rank < 2 || rank > 4)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "rank should be 2, 3 or 4");
    std::vector<index_t> out_shape;
    for (int d : dims_) {
      if (d < 0 || static_cast<size_t>(d) >= rank) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "bad dims");
      out_shape.push_back(in_shape[d]);
    }
    MACE_RETURN_IF_ERROR(output->Resize(out_shape));
    output->SetScale(input->scale());
    output->SetZeroPoint(input->zero_point());
    // dims_ = (0 .. b-1) (b+k .. rank-1) (b .. b+k-1)
    size_t b = 0;
    while (b < rank && dims_[b] == static_cast<int>(b)) ++b;
    CudaRuntime *rt = CudaRuntimeOf(context);
    if (b == rank)
      return rt->Status(mb_memcpy_d2d(rt->ctx(), output->mutable_memory<void>(), input->memory<void>(),
                                      static_cast<size_t>(input->raw_size())));
    const size_t first = static_cast<size_t>(dims_[b]);  // = b + k
    bool rotation = first > b;
    for (size_t i = b; i < rank && rotation; ++i) {
      const size_t want = i - b < rank - first ? first + (i - b) : b + (i - b) - (rank - first);
      rotation = static_cast<size_t>(dims_[i]) == want;
    }
    if (!rotation) return MaceStatus(MaceStatus::MACE_UNSUPPORTED, "Transpose: permutation is not a batched 2-D transpose");
    index_t batch = 1, rows = 1, cols = 1;
    for (size_t i = 0; i < b; ++i) batch *= in_shape[i];
    for (size_t i = b; i < first; ++i) rows *= in_shape[i];
    for (size_t i = first; i < rank; ++i) cols *= in_shape[i];
    return rt->Status(mb_transpose2d_batched(rt->ctx(), input->memory<void>(), output->mutable_memory<void>(), batch,
                                             rows, cols, static_cast<int>(sizeof(T))));
  }

 private:
  std::vector<int> dims_;
};

// Squeeze (mace/ops/squeeze.cc:25-84) and Reshape (mace/ops/reshape.cc:27-133).  The CPU
// operators let the output reuse the input's buffer; here the output keeps memory of its own
// and the bytes are copied on the device, so that the shared-memory plan, which frees a buffer
// after its tensor's last reader, never sees two tensors in one buffer.
template <RuntimeType D, class T>
class SqueezeOp : public Operation {
 public:
  explicit SqueezeOp(OpConstructContext *context)
      : Operation(context), axis_(GetRepeatedArgs<int>("axis", {})), checked_(false) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0);
    Tensor *output = Output(0);
    if (!checked_ && !std::is_same<T, uint8_t>::value) {
      // float tensors of this runtime are NCHW like the CPU runtime's: axes given for NHWC move
      if (GetOptionalArg<int>("has_data_format", 0) != 0 && input->dim_size() == 4 && axis_.size() == 2 &&
          axis_[0] == 1 && axis_[1] == 2) {
        axis_[0] = 2;
        axis_[1] = 3;
      }
      checked_ = true;
    }
    std::vector<index_t> out_shape;
    for (index_t i = 0; i < input->dim_size(); ++i) {
      const bool listed = std::find(axis_.begin(), axis_.end(), static_cast<int>(i)) != axis_.end();
      if (input->dim(static_cast<unsigned>(i)) > 1 || (!axis_.empty() && !listed))
        out_shape.push_back(input->dim(static_cast<unsigned>(i)));
    }
    MACE_RETURN_IF_ERROR(output->Resize(out_shape));
    output->SetScale(input->scale());
    output->SetZeroPoint(input->zero_point());
    CudaRuntime *rt = CudaRuntimeOf(context);
    return rt->Status(mb_memcpy_d2d(rt->ctx(), output->mutable_memory<void>(), input->memory<void>(),
                                    static_cast<size_t>(input->raw_size())));
  }

 private:
  std::vector<int> axis_;
  bool checked_;
};

template <RuntimeType D, class T>
class ReshapeOp : public Operation {
 public:
  explicit ReshapeOp(OpConstructContext *context)
      : Operation(context), dim_(GetRepeatedArgs<int>("dim", {})),
        has_df_(GetOptionalArg<int>("has_data_format", 0) != 0) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0);
    Tensor *output = Output(0);
    CudaRuntime *rt = CudaRuntimeOf(context);
    if (dim_.empty()) {
      // the shape tensor (int32, a constant of the model) is read back once
      if (InputSize() < 2) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Reshape needs a dim argument or a shape input");
      const Tensor *shape = Input(1);
      if (shape->dtype() != DT_INT32) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Reshape: the shape input must be int32");
      std::vector<int32_t> host(static_cast<size_t>(shape->size()));
      MACE_RETURN_IF_ERROR(rt->Status(mb_memcpy_d2h(rt->ctx(), host.data(), shape->memory<void>(),
                                                    static_cast<size_t>(shape->raw_size()))));
      MACE_RETURN_IF_ERROR(rt->Status(mb_stream_sync(rt->ctx())));
      dim_.assign(host.begin(), host.end());
    }
    std::vector<int> target = dim_;
    if (has_df_ && !std::is_same<T, uint8_t>::value && target.size() == 4)
      target = {target[0], target[3], target[1], target[2]};  // NHWC -> NCHW
    // GetOutputShape (reshape.cc:27-69): one -1 is inferred, 0 keeps the input's extent
    std::vector<index_t> out_shape(target.size());
    index_t product = 1;
    int unknown = -1;
    for (size_t i = 0; i < target.size(); ++i) {
      if (target[i] == -1) {
        if (unknown != -1) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Only one input size may be -1");
        unknown = static_cast<int>(i);
        out_shape[i] = 1;
      } else if (target[i] == 0) {
        if (static_cast<index_t>(i) >= input->dim_size())
          return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "dims:0 out of input dims' range.");
        out_shape[i] = input->dim(static_cast<unsigned>(i));
        product *= out_shape[i];
      } else {
        if (target[i] < 0) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Shape must be non-negative");
        out_shape[i] = target[i];
        product *= target[i];
      }
    }
    if (unknown != -1) {
      if (product == 0) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Cannot infer shape if there is zero shape size.");
      const index_t missing = input->size() / product;
      if (missing * product != input->size())
        return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Input size not match reshaped tensor size");
      out_shape[static_cast<size_t>(unknown)] = missing;
      product *= missing;
    }
    if (product != input->size()) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Input size not match reshaped tensor size");
    MACE_RETURN_IF_ERROR(output->Resize(out_shape));
    output->SetScale(input->scale());
    output->SetZeroPoint(input->zero_point());
    return rt->Status(mb_memcpy_d2d(rt->ctx(), output->mutable_memory<void>(), input->memory<void>(),
                                    static_cast<size_t>(input->raw_size())));
  }

 private:
  std::vector<int> dim_;
  bool has_df_;
};

// Internal to this runtime (no MACE operator of this name): the pixels a strided 1x1
// convolution reads, see SerialNet::ShareSubsampledInputs.  Argument "strides".
template <RuntimeType D, class T>
class SubsampleOp : public Operation {
 public:
  explicit SubsampleOp(OpConstructContext *context)
      : Operation(context), strides_(GetRepeatedArgs<int>("strides", {1, 1})) {}

  MaceStatus Run(OpContext *context) override {
    const Tensor *input = Input(0);
    Tensor *output = Output(0);
    if (input->dim_size() != 4 || strides_.size() != 2 || strides_[0] < 1 || strides_[1] < 1)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "Subsample needs a 4-D input and two strides");
    const index_t H = input->dim(2), W = input->dim(3);
    MACE_RETURN_IF_ERROR(output->Resize({input->dim(0), input->dim(1), (H + strides_[0] - 1) / strides_[0],
                                         (W + strides_[1] - 1) / strides_[1]}));
    CudaRuntime *rt = CudaRuntimeOf(context);
    return rt->Status(mb_subsample_f32_nchw(rt->ctx(), input->memory<float>(), output->mutable_memory<float>(),
                                            input->dim(0) * input->dim(1), H, W, strides_[0], strides_[1]));
  }

 private:
  std::vector<int> strides_;
};

#define MACE_REGISTER_OP(registry, op_type, class_name, runtime, dt)                             \
  registry->Register(op_type, runtime, DataTypeToEnum<dt>::value,                                \
                     [](OpConstructContext *context) -> std::unique_ptr<Operation> {             \
                       return std::unique_ptr<Operation>(new class_name<runtime, dt>(context));  \
                     })

void RegisterAllCudaOps(OpRegistry *registry) {
  MACE_REGISTER_OP(registry, "Conv2D", Conv2dOp, RuntimeType::RT_CUDA, uint8_t);
  MACE_REGISTER_OP(registry, "DepthwiseConv2d", DepthwiseConv2dOp, RuntimeType::RT_CUDA, uint8_t);
  MACE_REGISTER_OP(registry, "MatMul", MatMulOp, RuntimeType::RT_CUDA, uint8_t);
  MACE_REGISTER_OP(registry, "FullyConnected", FullyConnectedOp, RuntimeType::RT_CUDA, uint8_t);
  MACE_REGISTER_OP(registry, "Pooling", PoolingOp, RuntimeType::RT_CUDA, uint8_t);
  MACE_REGISTER_OP(registry, "Conv2D", Conv2dOp, RuntimeType::RT_CUDA, float);
  MACE_REGISTER_OP(registry, "DepthwiseConv2d", DepthwiseConv2dOp, RuntimeType::RT_CUDA, float);
  MACE_REGISTER_OP(registry, "MatMul", MatMulOp, RuntimeType::RT_CUDA, float);
  MACE_REGISTER_OP(registry, "FullyConnected", FullyConnectedOp, RuntimeType::RT_CUDA, float);
  MACE_REGISTER_OP(registry, "Pooling", PoolingOp, RuntimeType::RT_CUDA, float);
  MACE_REGISTER_OP(registry, "Eltwise", EltwiseOp, RuntimeType::RT_CUDA, float);
  MACE_REGISTER_OP(registry, "Activation", ActivationOp, RuntimeType::RT_CUDA, float);
  MACE_REGISTER_OP(registry, "Softmax", SoftmaxOp, RuntimeType::RT_CUDA, float);
  MACE_REGISTER_OP(registry, "Quantize", QuantizeOp, RuntimeType::RT_CUDA, uint8_t);
  MACE_REGISTER_OP(registry, "Dequantize", DequantizeOp, RuntimeType::RT_CUDA, uint8_t);
  MACE_REGISTER_OP(registry, "Dequantize", DequantizeOp, RuntimeType::RT_CUDA, int32_t);
  MACE_REGISTER_OP(registry, "Transpose", TransposeOp, RuntimeType::RT_CUDA, float);
  MACE_REGISTER_OP(registry, "Transpose", TransposeOp, RuntimeType::RT_CUDA, uint8_t);
  MACE_REGISTER_OP(registry, "Squeeze", SqueezeOp, RuntimeType::RT_CUDA, float);
  MACE_REGISTER_OP(registry, "Squeeze", SqueezeOp, RuntimeType::RT_CUDA, uint8_t);
  MACE_REGISTER_OP(registry, "Reshape", ReshapeOp, RuntimeType::RT_CUDA, float);
  MACE_REGISTER_OP(registry, "Reshape", ReshapeOp, RuntimeType::RT_CUDA, uint8_t);
  MACE_REGISTER_OP(registry, "Subsample", SubsampleOp, RuntimeType::RT_CUDA, float);
}

}  // namespace ops

// ---- SerialNet -------------------------------------------------------------------

namespace {
void DescribeOperator(Operation *op, OperatorStats *os);
}

MaceStatus SerialNet::AddOperator(const OperatorDef &def) {
  DropCapture();
  defs_.push_back(std::make_unique<OperatorDef>(def));
  const OperatorDef *d = defs_.back().get();
  OpConstructContext cc(ws_, runtime_, d);
  auto it = d->i.find("T");
  const DataType dt = it == d->i.end() ? DT_FLOAT : static_cast<DataType>(it->second);
  MaceStatus st;
  std::unique_ptr<Operation> op = op_registry_->CreateOperation(&cc, RuntimeType::RT_CUDA, dt, &st);
  if (op == nullptr) {
    defs_.pop_back();
    return st;
  }
  st = op->Init(&cc);
  if (st != MaceStatus::MACE_SUCCESS) {
    defs_.pop_back();
    return st;
  }
  operators_.push_back(std::move(op));
  skipped_.push_back(0);
  return MaceStatus::MACE_SUCCESS;
}

int SerialNet::FuseActivations(const std::set<std::string> *keep) {
  DropCapture();
  std::map<std::string, int> readers;
  for (const auto &d : defs_)
    for (const std::string &in : d->input) ++readers[in];
  int merged = 0;
  for (size_t a = 0; a < defs_.size(); ++a) {
    if (skipped_[a] || defs_[a]->type != "Activation" || defs_[a]->input.empty()) continue;
    const std::string &mid = defs_[a]->input[0];
    if (readers[mid] != 1 || (keep != nullptr && keep->count(mid) != 0)) continue;
    for (size_t pr = 0; pr < a; ++pr) {
      if (skipped_[pr] || defs_[pr]->output.size() != 1 || defs_[pr]->output[0] != mid) continue;
      if (operators_[pr]->AbsorbActivation(*defs_[a], operators_[a]->Output(0))) {
        skipped_[a] = 1;
        ++merged;
      }
      break;
    }
  }
  return merged;
}

int SerialNet::FuseResidualSums(const std::set<std::string> *keep) {
  DropCapture();
  std::map<std::string, int> readers;
  std::map<std::string, size_t> producer;
  for (size_t i = 0; i < defs_.size(); ++i) {
    if (skipped_[i]) continue;
    for (const std::string &in : defs_[i]->input) ++readers[in];
    // the tensor an operator really writes (it may have taken over a later operator's output)
    for (size_t k = 0; k < defs_[i]->output.size(); ++k)
      producer[operators_[i]->Output(static_cast<unsigned>(k))->name()] = i;
  }
  int merged = 0;
  for (size_t e = 0; e < defs_.size(); ++e) {
    if (skipped_[e]) continue;
    Operation::ResidualSum sum;
    if (!operators_[e]->DescribeResidualSum(&sum)) continue;
    for (int side = 0; side < 2; ++side) {
      const Tensor *conv_out = operators_[e]->Input(side), *residual = operators_[e]->Input(1 - side);
      auto pc = producer.find(conv_out->name());
      if (pc == producer.end() || pc->second >= e || readers[conv_out->name()] != 1) continue;
      if (keep != nullptr && keep->count(conv_out->name()) != 0) continue;
      if (defs_[pc->second]->type != "Conv2D") continue;
      // the residual must exist when the convolution runs: a net input, a weight, or produced earlier
      auto pr = producer.find(residual->name());
      if (pr != producer.end() && pr->second >= pc->second) continue;
      if (operators_[pc->second]->AbsorbResidualSum(residual, sum, operators_[e]->Output(0))) {
        skipped_[e] = 1;
        ++merged;
        break;
      }
    }
  }
  return merged;
}

int SerialNet::ShareSubsampledInputs() {
  DropCapture();
  // members of each (input tensor, strides) group, in net order
  std::map<std::string, std::vector<size_t>> groups;
  std::map<std::string, std::pair<int, int>> group_strides;
  for (size_t i = 0; i < operators_.size(); ++i) {
    int sh = 0, sw = 0;
    if (skipped_[i] || defs_[i]->input.empty() || !operators_[i]->DescribeStridedPointwise(&sh, &sw)) continue;
    const std::string key = defs_[i]->input[0] + "/subsampled_" + std::to_string(sh) + "x" + std::to_string(sw);
    groups[key].push_back(i);
    group_strides[key] = {sh, sw};
  }
  std::vector<Operation *> member_ops(operators_.size());
  std::vector<OperatorDef *> member_defs(operators_.size());
  for (size_t i = 0; i < operators_.size(); ++i) {
    member_ops[i] = operators_[i].get();
    member_defs[i] = defs_[i].get();
  }
  // the new operators are inserted from the back of the net, so that earlier positions stay valid
  std::vector<std::pair<size_t, std::string>> order;
  for (const auto &kv : groups)
    if (kv.second.size() >= 2) order.emplace_back(kv.second.front(), kv.first);
  std::sort(order.begin(), order.end(), [](const auto &a, const auto &b) { return a.first > b.first; });
  int shared = 0;
  for (const auto &entry : order) {
    // (pointers, not indices: an insertion further back has moved the members behind it)
    std::vector<std::pair<Operation *, OperatorDef *>> members;
    for (size_t m : groups[entry.second]) members.emplace_back(member_ops[m], member_defs[m]);
    auto def = std::make_unique<OperatorDef>();
    def->type = "Subsample";
    def->name = entry.second;
    def->input = {members.front().second->input[0]};
    def->output = {entry.second};
    def->ints["strides"] = {group_strides[entry.second].first, group_strides[entry.second].second};
    def->i["T"] = static_cast<int>(DT_FLOAT);
    OpConstructContext cc(ws_, runtime_, def.get());
    MaceStatus st;
    std::unique_ptr<Operation> op = op_registry_->CreateOperation(&cc, RuntimeType::RT_CUDA, DT_FLOAT, &st);
    if (op == nullptr || op->Init(&cc) != MaceStatus::MACE_SUCCESS) continue;
    for (const auto &m : members) {
      m.first->TakeSubsampledInput(op->Output(0));
      m.second->input[0] = entry.second;
      m.second->ints["strides"] = {1, 1};
    }
    const auto at = static_cast<std::ptrdiff_t>(entry.first);
    defs_.insert(defs_.begin() + at, std::move(def));
    operators_.insert(operators_.begin() + at, std::move(op));
    skipped_.insert(skipped_.begin() + at, 0);
    ++shared;
  }
  return shared;
}

SerialNet::~SerialNet() {
  DropCapture();
  operators_.clear();  // delegators may hold device memory; tensors are the workspace's
  for (void *b : shared_buffers_) runtime_->Delete(b);
}

MaceStatus SerialNet::PlanMemory(size_t *separate_bytes, size_t *shared_bytes, const std::set<std::string> *keep) {
  DropCapture();
  struct Ref {
    Tensor *tensor;
    int refs = 0;
    int buffer = -1;
    bool produced = false;
  };
  std::map<std::string, Ref> refs;
  // readers of every activation tensor
  for (size_t i = 0; i < operators_.size(); ++i) {
    if (skipped_[i]) continue;
    for (int k = 0; k < operators_[i]->InputSize(); ++k) {
      const Tensor *t = operators_[i]->Input(k);
      if (t->is_weight()) continue;
      Ref &r = refs[t->name()];
      r.tensor = const_cast<Tensor *>(t);
      r.refs++;
    }
  }
  struct Buf {
    size_t bytes;
    bool free;
  };
  std::vector<Buf> bufs;
  size_t separate = 0;
  for (size_t i = 0; i < operators_.size(); ++i) {
    if (skipped_[i]) continue;
    const OperatorDef &def = operators_[i]->debug_def();
    for (size_t k = 0; k < def.output.size(); ++k) {
      Tensor *t = operators_[i]->Output(static_cast<unsigned>(k));
      auto it = refs.find(t->name());
      if (it == refs.end()) continue;  // nobody reads it: an output of the net, keeps its memory
      if (keep != nullptr && keep->count(t->name()) != 0) continue;  // a named output that is also read
      Ref &r = it->second;
      if (r.produced) continue;        // written by two operators: first placement stands
      r.produced = true;
      const size_t need = static_cast<size_t>(t->raw_size());
      if (need == 0)
        return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "PlanMemory: run the net once first (tensor " +
                                                             t->name() + " has no shape)");
      separate += need;
      // best fit: the smallest free buffer that is large enough, else the largest free one, grown
      int best = -1;
      for (size_t b = 0; b < bufs.size(); ++b) {
        if (!bufs[b].free) continue;
        if (best < 0) { best = static_cast<int>(b); continue; }
        const bool fits = bufs[b].bytes >= need, best_fits = bufs[best].bytes >= need;
        if (fits && (!best_fits || bufs[b].bytes < bufs[best].bytes)) best = static_cast<int>(b);
        else if (!fits && !best_fits && bufs[b].bytes > bufs[best].bytes) best = static_cast<int>(b);
      }
      if (best < 0) {
        bufs.push_back({need, false});
        best = static_cast<int>(bufs.size()) - 1;
      } else {
        bufs[best].free = false;
        bufs[best].bytes = std::max(bufs[best].bytes, need);
      }
      r.buffer = best;
    }
    for (int k = 0; k < operators_[i]->InputSize(); ++k) {
      const Tensor *t = operators_[i]->Input(k);
      if (t->is_weight()) continue;
      Ref &r = refs[t->name()];
      if (--r.refs == 0 && r.buffer >= 0) bufs[r.buffer].free = true;  // (net inputs have no buffer)
    }
  }
  // allocate the shared buffers and move the tensors in
  std::vector<void *> mem(bufs.size(), nullptr);
  size_t shared = 0;
  for (size_t b = 0; b < bufs.size(); ++b) {
    MACE_RETURN_IF_ERROR(runtime_->New(bufs[b].bytes, &mem[b]));
    shared_buffers_.push_back(mem[b]);
    shared += bufs[b].bytes;
  }
  for (auto &kv : refs)
    if (kv.second.buffer >= 0) kv.second.tensor->BindShared(mem[kv.second.buffer], bufs[kv.second.buffer].bytes);
  if (separate_bytes != nullptr) *separate_bytes = separate;
  if (shared_bytes != nullptr) *shared_bytes = shared;
  return MaceStatus::MACE_SUCCESS;
}

MaceStatus SerialNet::Capture() {
  DropCapture();
  OpContext context(runtime_);
  // one graph, or two when an input is watched: [0, watch_index_] and the rest
  const size_t n = operators_.size();
  const size_t cut = (watch_event_ != nullptr && watch_index_ >= 0 && static_cast<size_t>(watch_index_) + 1 < n)
                         ? static_cast<size_t>(watch_index_) + 1
                         : n;
  void *graphs[2] = {nullptr, nullptr};
  MaceStatus st = MaceStatus::MACE_SUCCESS;
  for (int part = 0; part < 2 && st == MaceStatus::MACE_SUCCESS; ++part) {
    const size_t begin = part == 0 ? 0 : cut, end_op = part == 0 ? cut : n;
    if (begin >= end_op) continue;
    st = runtime_->Status(mb_graph_begin(runtime_->ctx()));
    if (st != MaceStatus::MACE_SUCCESS) break;
    for (size_t i = begin; i < end_op && st == MaceStatus::MACE_SUCCESS; ++i)
      if (!skipped_[i]) st = operators_[i]->Run(&context);
    MaceStatus end = runtime_->Status(mb_graph_end(runtime_->ctx(), &graphs[part]));
    if (st == MaceStatus::MACE_SUCCESS) st = end;
  }
  if (st != MaceStatus::MACE_SUCCESS) {
    for (void *g : graphs)
      if (g != nullptr) mb_graph_destroy(runtime_->ctx(), g);
    return st;
  }
  graph_ = graphs[0];
  graph_tail_ = graphs[1];
  return MaceStatus::MACE_SUCCESS;
}

MaceStatus SerialNet::WatchInput(const std::string &input_name, void *event) {
  int last = -1;
  if (event != nullptr) {
    for (size_t i = 0; i < defs_.size(); ++i) {
      if (skipped_[i]) continue;
      for (const std::string &in : defs_[i]->input)
        if (in == input_name) last = static_cast<int>(i);
    }
    if (last < 0) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "no operator of the net reads " + input_name);
  }
  if (last == watch_index_ && event == watch_event_) return MaceStatus::MACE_SUCCESS;
  const bool was_captured = captured();
  watch_index_ = last;
  watch_event_ = event;
  if (was_captured) return Capture();  // the split point moved
  return MaceStatus::MACE_SUCCESS;
}

MaceStatus SerialNet::RunProfiledGraph(RunMetadata *run_metadata, int replays) {
  if (run_metadata == nullptr || replays < 1) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "RunProfiledGraph");
  mb_context *ctx = runtime_->ctx();
  OpContext context(runtime_);
  std::vector<void *> events(operators_.size() + 1, nullptr);
  MaceStatus st = MaceStatus::MACE_SUCCESS;
  for (auto &e : events)
    if (st == MaceStatus::MACE_SUCCESS) st = runtime_->Status(mb_event_create(ctx, &e));
  void *graph = nullptr;
  if (st == MaceStatus::MACE_SUCCESS) st = runtime_->Status(mb_graph_begin(ctx));
  if (st == MaceStatus::MACE_SUCCESS) {
    st = runtime_->Status(mb_event_record(ctx, events[0]));
    for (size_t i = 0; i < operators_.size() && st == MaceStatus::MACE_SUCCESS; ++i) {
      if (!skipped_[i]) st = operators_[i]->Run(&context);
      if (st == MaceStatus::MACE_SUCCESS) st = runtime_->Status(mb_event_record(ctx, events[i + 1]));
    }
    MaceStatus end = runtime_->Status(mb_graph_end(ctx, &graph));
    if (st == MaceStatus::MACE_SUCCESS) st = end;
  }
  std::vector<float> total(operators_.size(), 0.f);
  for (int r = 0; r <= replays && st == MaceStatus::MACE_SUCCESS; ++r) {  // replay 0 warms up
    st = runtime_->Status(mb_graph_launch(ctx, graph));
    if (st == MaceStatus::MACE_SUCCESS) st = runtime_->Status(mb_stream_sync(ctx));
    for (size_t i = 0; i < operators_.size() && st == MaceStatus::MACE_SUCCESS && r > 0; ++i) {
      float ms = 0.f;
      st = runtime_->Status(mb_event_elapsed_ms(ctx, events[i], events[i + 1], &ms));
      total[i] += ms;
    }
  }
  if (st == MaceStatus::MACE_SUCCESS) {
    run_metadata->op_stats.clear();
    float since_start = 0.f;
    for (size_t i = 0; i < operators_.size(); ++i) {
      OperatorStats os;
      DescribeOperator(operators_[i].get(), &os);
      os.device_ms = total[i] / static_cast<float>(replays);
      os.stats.start_micros = static_cast<int64_t>(since_start * 1000.f + 0.5f);
      since_start += os.device_ms;
      os.stats.end_micros = static_cast<int64_t>(since_start * 1000.f + 0.5f);
      run_metadata->op_stats.push_back(os);
    }
  }
  if (graph != nullptr) mb_graph_destroy(ctx, graph);
  for (auto &e : events)
    if (e != nullptr) mb_event_destroy(ctx, e);
  return st;
}

void SerialNet::DropCapture() {
  if (graph_ != nullptr) {
    mb_graph_destroy(runtime_->ctx(), graph_);
    graph_ = nullptr;
  }
  if (graph_tail_ != nullptr) {
    mb_graph_destroy(runtime_->ctx(), graph_tail_);
    graph_tail_ = nullptr;
  }
}

namespace {

// What the reference records about an operator next to its times (serial_net.cc:138-180).
void DescribeOperator(Operation *op, OperatorStats *os) {
  const OperatorDef &def = op->debug_def();
  os->operator_name = def.name;
  os->type = def.type;
  const std::string &type = def.type;
  if (type == "Conv2D" || type == "Deconv2D" || type == "DepthwiseConv2d" || type == "DepthwiseDeconv2d" ||
      type == "Pooling") {
    os->args.strides = op->GetRepeatedArgs<int>("strides");
    os->args.padding_type = op->GetOptionalArg<int>("padding", -1);
    os->args.paddings = op->GetRepeatedArgs<int>("padding_values");
    os->args.dilations = op->GetRepeatedArgs<int>("dilations");
    if (type == "Pooling") {
      for (int k : op->GetRepeatedArgs<int>("kernels")) os->args.kernels.push_back(k);
    } else if (op->InputSize() >= 2) {
      os->args.kernels = op->Input(1)->shape();
    }
  } else if (type == "MatMul") {
    os->args.kernels = op->Input(0)->shape();
    if (op->GetOptionalArg<bool>("transpose_a", false) && os->args.kernels.size() >= 2)
      std::swap(os->args.kernels[os->args.kernels.size() - 2], os->args.kernels[os->args.kernels.size() - 1]);
  } else if (type == "FullyConnected" && op->InputSize() >= 2) {
    os->args.kernels = op->Input(1)->shape();
  }
  for (const Tensor *t : op->Outputs()) os->output_shape.push_back(t->shape());
}

std::string ShapeString(const std::vector<index_t> &shape) {
  std::ostringstream ss;
  ss << "[";
  for (size_t i = 0; i < shape.size(); ++i) ss << (i ? ", " : "") << shape[i];
  ss << "]";
  return ss.str();
}

// serial_net.cc:185-224: the ranges of an operator's outputs, reduced on the device.
MaceStatus LogTensorRanges(CudaRuntime *runtime, Operation *op) {
  const OperatorDef &def = op->debug_def();
  for (int i = 0; i < op->OutputSize(); ++i) {
    const Tensor *out = op->Output(i);
    const std::string &name = static_cast<size_t>(i) < def.output.size() ? def.output[i] : out->name();
    if (out->dtype() != DT_FLOAT)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS,
                        "On quantize_stat mode, must use float32 model (tensor " + name + ")");
    if (def.quantize_info.empty()) {
      float min_v = 0.f, max_v = 0.f;
      MACE_RETURN_IF_ERROR(runtime->Status(mb_minmax_f32(runtime->ctx(), out->memory<float>(), out->size(),
                                                         &min_v, &max_v)));
      LOG(INFO) << "Tensor range @@" << name << "@@" << min_v << "," << max_v;
    } else {
      const int bin_size = 2048;
      for (const QuantizeActivationInfo &q : def.quantize_info) {
        std::vector<int32_t> bins(bin_size, 0);
        MACE_RETURN_IF_ERROR(runtime->Status(mb_histogram_f32(runtime->ctx(), out->memory<float>(), out->size(),
                                                              q.minval, q.maxval, bin_size, bins.data())));
        std::ostringstream ss;
        ss << "[";
        for (int b = 0; b < bin_size; ++b) ss << (b ? ", " : "") << bins[b];
        ss << "]";
        LOG(INFO) << "Tensor range @@" << name << "@@" << q.minval << "," << q.maxval << "@@" << ss.str();
      }
    }
  }
  return MaceStatus::MACE_SUCCESS;
}

}  // namespace

MaceStatus SerialNet::Run(RunMetadata *run_metadata) {
  const bool log_ranges = EnvConfEnabled("MACE_LOG_TENSOR_RANGE");
  MACE_LATENCY_LOGGER(1, "Running net");
  void *wait_event = wait_event_;
  wait_event_ = nullptr;
  const bool watching = watch_event_ != nullptr && watch_index_ >= 0;
  if (wait_event != nullptr && !watching)
    MACE_RETURN_IF_ERROR(runtime_->Status(mb_stream_wait_event(runtime_->ctx(), wait_event)));
  if (graph_ != nullptr && run_metadata == nullptr && !log_ranges) {
    MACE_RETURN_IF_ERROR(runtime_->Status(mb_graph_launch(runtime_->ctx(), graph_)));
    if (watch_event_ != nullptr) MACE_RETURN_IF_ERROR(runtime_->Status(mb_event_record(runtime_->ctx(), watch_event_)));
    if (wait_event != nullptr && watching)
      MACE_RETURN_IF_ERROR(runtime_->Status(mb_stream_wait_event(runtime_->ctx(), wait_event)));
    if (graph_tail_ != nullptr) MACE_RETURN_IF_ERROR(runtime_->Status(mb_graph_launch(runtime_->ctx(), graph_tail_)));
    return MaceStatus::MACE_SUCCESS;
  }
  OpContext context(runtime_);
  std::vector<void *> events;
  if (run_metadata != nullptr) {
    events.resize(operators_.size() + 1, nullptr);
    for (auto &e : events) MACE_RETURN_IF_ERROR(runtime_->Status(mb_event_create(runtime_->ctx(), &e)));
    MACE_RETURN_IF_ERROR(runtime_->Status(mb_event_record(runtime_->ctx(), events[0])));
  }
  MaceStatus st = MaceStatus::MACE_SUCCESS;
  for (size_t i = 0; i < operators_.size() && st == MaceStatus::MACE_SUCCESS; ++i) {
    Operation *op = operators_[i].get();
    if (!skipped_[i]) {
      MACE_LATENCY_LOGGER(2, "Running operator " + op->debug_def().name + "<CUDA, " + op->debug_def().type + ">");
      st = op->Run(&context);
      if (st != MaceStatus::MACE_SUCCESS) {
        VLOG(0) << "operator " << op->debug_def().name << " (" << op->debug_def().type
                << ") failed with error: " << st.information();
        break;
      }
      VLOG(3) << "Operator " << op->debug_def().name << " has shape: " << ShapeString(op->Output(0)->shape());
      if (log_ranges) st = LogTensorRanges(runtime_, op);
    }
    if (watch_event_ != nullptr && static_cast<int>(i) == watch_index_ && st == MaceStatus::MACE_SUCCESS) {
      st = runtime_->Status(mb_event_record(runtime_->ctx(), watch_event_));
      if (wait_event != nullptr && st == MaceStatus::MACE_SUCCESS)
        st = runtime_->Status(mb_stream_wait_event(runtime_->ctx(), wait_event));
    }
    if (run_metadata != nullptr && st == MaceStatus::MACE_SUCCESS)
      st = runtime_->Status(mb_event_record(runtime_->ctx(), events[i + 1]));
  }
  if (run_metadata != nullptr && st == MaceStatus::MACE_SUCCESS) {
    run_metadata->op_stats.clear();
    float since_start = 0.f;
    for (size_t i = 0; i < operators_.size() && st == MaceStatus::MACE_SUCCESS; ++i) {
      OperatorStats os;
      DescribeOperator(operators_[i].get(), &os);
      st = runtime_->Status(mb_event_elapsed_ms(runtime_->ctx(), events[i], events[i + 1], &os.device_ms));
      os.stats.start_micros = static_cast<int64_t>(since_start * 1000.f + 0.5f);
      since_start += os.device_ms;
      os.stats.end_micros = static_cast<int64_t>(since_start * 1000.f + 0.5f);
      run_metadata->op_stats.push_back(os);
    }
  }
  for (auto &e : events)
    if (e != nullptr) mb_event_destroy(runtime_->ctx(), e);
  return st;
}

}  // namespace mace
