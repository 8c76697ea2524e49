// Operators for RuntimeType::RT_CUDA with the argument names and Run() behaviour of MACE's CPU
// operators:
//   uint8   Conv2dOp            mace/ops/conv_2d.cc:190-318     (inputs INPUT, FILTER, BIAS)
//           DepthwiseConv2dOp   mace/ops/depthwise_conv2d.cc:146-250
//           MatMulOp            mace/ops/matmul.cc:397-482      (args transpose_a, transpose_b)
//           FullyConnectedOp    mace/ops/fully_connected.cc:130-179
//           PoolingOp (AVG)     mace/ops/pooling.cc:638-871     (args kernels, pooling_type, round_mode)
//           QuantizeOp, DequantizeOp   mace/ops/quantize.cc:31-115
//   float   Conv2dOp (mace/ops/conv_2d.cc:82-176), DepthwiseConv2dOp, MatMulOp, FullyConnectedOp,
//           PoolingOp (mace/ops/pooling.cc:46-240), EltwiseOp (mace/ops/eltwise.cc:949-1144),
//           ActivationOp (mace/ops/activation.cc:36-79), SoftmaxOp (mace/ops/softmax.cc:249-290)
//   both    TransposeOp (mace/ops/transpose.cc:34-73), SqueezeOp (mace/ops/squeeze.cc:25-84),
//           ReshapeOp (mace/ops/reshape.cc:27-133)
// plus the sequential executor (SerialNet::Run, mace/core/net/serial_net.cc:93-228) with
// activation merging and MACE's shared activation memory
// (mace/core/net/allocate_opt_strategy.cc:181-285), and a small OperatorDef stand-in
// (mace/proto/mace.proto:61-95: type, inputs, outputs, args, output_type, quantize_info).
#ifndef MACE_B200_HOST_OPS_H_
#define MACE_B200_HOST_OPS_H_

#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "core.h"
#include "delegators.h"

namespace mace {

struct QuantizeActivationInfo {  // mace.proto:61-66
  float scale = 0.f;
  int32_t zero_point = 0;
  float minval = 0.f;  // the range a quantize-aware training run recorded (used by range logging)
  float maxval = 0.f;
};

struct OperatorDef {
  std::string type;
  std::string name;
  std::vector<std::string> input;
  std::vector<std::string> output;
  std::map<std::string, std::vector<int>> ints;   // "strides", "dilations", "padding_values", "kernels"
  std::map<std::string, int> i;                   // "padding", "transpose_a", "T", "pooling_type", ...
  std::map<std::string, float> f;                 // "max_limit", ...
  std::map<std::string, std::vector<float>> floats;  // "coeff"
  std::map<std::string, std::string> s;           // "activation"
  std::vector<DataType> output_type;
  std::vector<QuantizeActivationInfo> quantize_info;
};

// Per-operator statistics of one run, the types of include/mace/public/mace.h:177-201.  Here the
// times come from CUDA events on the runtime's stream: start_micros / end_micros are device time
// since the net's first operator was enqueued (rounded to microseconds), device_ms (an
// addition) keeps the event resolution.
struct CallStats {
  int64_t start_micros = 0;
  int64_t end_micros = 0;
};

struct ConvPoolArgs {
  std::vector<int> strides;
  int padding_type = -1;
  std::vector<int> paddings;
  std::vector<int> dilations;
  std::vector<int64_t> kernels;
};

struct OperatorStats {
  std::string operator_name;
  std::string type;
  std::vector<std::vector<int64_t>> output_shape;
  ConvPoolArgs args;
  CallStats stats;
  float device_ms = 0.f;
};

class RunMetadata {
 public:
  std::vector<OperatorStats> op_stats;
};

class OpConstructContext {
 public:
  OpConstructContext(Workspace *ws, Runtime *rt, const OperatorDef *def)
      : workspace_(ws), runtime_(rt), operator_def_(def) {}
  Workspace *workspace() const { return workspace_; }
  Runtime *runtime() const { return runtime_; }
  const OperatorDef *operator_def() const { return operator_def_; }

 private:
  Workspace *workspace_;
  Runtime *runtime_;
  const OperatorDef *operator_def_;
};

class Operation {
 public:
  explicit Operation(OpConstructContext *context);
  virtual ~Operation() = default;

  template <typename T> T GetOptionalArg(const std::string &name, const T &default_value) const;
  template <typename T>
  std::vector<T> GetRepeatedArgs(const std::string &name, const std::vector<T> &default_value = {}) const;

  // Binds input and output tensors by name (Operation::Init, mace/core/ops/operator.cc:26-85):
  // outputs are created in the workspace with the output type and the
  // activation range of quantize_info.
  MaceStatus Init(OpConstructContext *context);
  virtual MaceStatus Run(OpContext *context) = 0;

  const Tensor *Input(unsigned int idx) const { return inputs_[idx]; }
  Tensor *Output(unsigned int idx) { return outputs_[idx]; }
  int InputSize() const { return static_cast<int>(inputs_.size()); }
  int OutputSize() const { return static_cast<int>(outputs_.size()); }
  const std::vector<Tensor *> &Outputs() const { return outputs_; }
  const OperatorDef &debug_def() const { return *operator_def_; }

  // Net-level merging of this operator with the Activation operator that consumes its only
  // output: an operator that can apply the activation itself takes it over, writes into
  // `activation_output` from then on and returns true; the net then skips the Activation.
  virtual bool AbsorbActivation(const OperatorDef &activation_def, Tensor *activation_output) {
    (void)activation_def;
    (void)activation_output;
    return false;
  }
  // An operator that is a plain sum of two tensors of equal size (no coefficients, no scalar)
  // describes itself here, with the activation it may already have absorbed, so that the
  // operator producing one of its inputs can take the whole thing over (AbsorbResidualSum).
  struct ResidualSum {
    int activation = 0;  // ops::ActivationType value
    float max_limit = 0.f, coefficient = 0.f;
  };
  virtual bool DescribeResidualSum(ResidualSum *sum) const {
    (void)sum;
    return false;
  }
  // out = activation(this operator's result + residual), written to `sum_output`: a convolution
  // that can add a residual in its own kernel returns true and does that from then on.
  // A float 1x1 convolution with a stride above 1, no dilation and no padding reads every
  // stride-th pixel only: it names its strides here, and TakeSubsampledInput() turns it into a
  // stride-1 convolution of `subsampled` (that tensor holds exactly those pixels), so that several
  // such convolutions of one tensor share one gather (SerialNet::ShareSubsampledInputs).
  virtual bool DescribeStridedPointwise(int *stride_h, int *stride_w) const {
    (void)stride_h;
    (void)stride_w;
    return false;
  }
  virtual void TakeSubsampledInput(const Tensor *subsampled) { (void)subsampled; }
  virtual bool AbsorbResidualSum(const Tensor *residual, const ResidualSum &sum, Tensor *sum_output) {
    (void)residual;
    (void)sum;
    (void)sum_output;
    return false;
  }

 protected:
  const OperatorDef *operator_def_;
  std::vector<const Tensor *> inputs_;
  std::vector<Tensor *> outputs_;
};

typedef std::function<std::unique_ptr<Operation>(OpConstructContext *)> OpCreator;

// Keyed by (type, runtime, data type) like MACE_REGISTER_OP
// (mace/core/registry/ops_registry.h:73-77).
class OpRegistry {
 public:
  MaceStatus Register(const std::string &type, RuntimeType rt, DataType dt, OpCreator creator);
  std::unique_ptr<Operation> CreateOperation(OpConstructContext *context, RuntimeType rt, DataType dt,
                                             MaceStatus *status) const;

 private:
  std::map<std::string, OpCreator> registry_;
};

namespace ops {
// Registers the operators listed at the top of this file.
void RegisterAllCudaOps(OpRegistry *registry);
}  // namespace ops

// Runs a list of operators in order on one CudaRuntime.
class SerialNet {
 public:
  SerialNet(const OpRegistry *op_registry, Workspace *ws, CudaRuntime *runtime)
      : op_registry_(op_registry), ws_(ws), runtime_(runtime) {}
  // The OperatorDef is copied; its tensors must exist (inputs) or are created (outputs).
  MaceStatus AddOperator(const OperatorDef &def);
  // run_metadata may be null; when given, each operator is bracketed by device
  // events and described as the reference describes it (mace/core/net/serial_net.cc:122-180).
  // With the environment switch MACE_LOG_TENSOR_RANGE on, every operator's outputs are reduced
  // on the device after it ran and logged as "Tensor range @@<name>@@<min>,<max>" (float models;
  // with a quantize_info range: plus the 2048-bin histogram), the lines the post-training
  // quantization tooling reads (serial_net.cc:185-224); a recorded graph is then not replayed.
  MaceStatus Run(RunMetadata *run_metadata = nullptr);
  // Records one pass over the operators into a CUDA graph; later Run() calls
  // without run_metadata replay it.  Call after at least one plain Run() (so
  // that scratch and cached operands exist) and again after any change of
  // tensor shapes or operators.
  MaceStatus Capture();
  void DropCapture();
  // Per-operator device times INSIDE a graph replay: records the operator chain into a second
  // graph with an event-record node behind every operator, replays it `replays` times and
  // averages the time between consecutive nodes.  Unlike Run(run_metadata) the operators are
  // launched the way the recorded graph launches them, so the times add up to the graph's
  // duration.  Call after at least one plain Run().
  MaceStatus RunProfiledGraph(RunMetadata *run_metadata, int replays = 5);
  // Merges every Activation operator into the operator that produces its input when that
  // operator can absorb it (the float Eltwise: a residual sum and its ReLU become one pass)
  // and nothing else reads the intermediate tensor, which is then no longer written.
  // Returns the number of merged pairs.  Off unless called: operator by operator the net
  // behaves like the CPU runtime's.
  // Tensors named in keep (a model's declared outputs) are always written.
  int FuseActivations(const std::set<std::string> *keep = nullptr);
  // After FuseActivations: merges each (Eltwise SUM [+ absorbed Activation]) into the float
  // Conv2D that produces one of its two inputs, when nothing else reads that input and the
  // other input (the residual) is produced earlier in the net; the convolution then writes
  // activation(conv + residual) straight into the sum's output.  Returns the number of merges.
  int FuseResidualSums(const std::set<std::string> *keep = nullptr);
  // Where two or more strided 1x1 float convolutions read the same tensor with the same strides
  // (a ResNet block's shortcut and its first convolution), a Subsample operator is put in front of
  // the first of them and they become stride-1 convolutions of its output: one gather of the
  // pixels instead of one per convolution.  Call before the first Run() or before the other
  // merging passes (the convolutions pick their delegators again).  Returns the number of groups.
  int ShareSubsampledInputs();
  // Shares activation memory between tensors whose lifetimes do not overlap, the way
  // AllocateTensorMemory<SERIAL_OPT> does (mace/core/net/allocate_opt_strategy.cc:181-285): the
  // net is walked once; every operator's outputs take the best-fitting free buffer (the
  // smallest that is large enough, else the largest one, grown) BEFORE the operator's inputs
  // are released, so an output never aliases an input of its own operator; a tensor's buffer
  // returns to the free list after its last reader.  Weights, tensors no operator of the net
  // produces (the net's inputs) and tensors no operator reads (its outputs) keep their own
  // memory.  Call after one plain Run(): the sizes are the ones that run produced.  Intermediate
  // tensors can no longer be read back afterwards.  separate_bytes / shared_bytes (may be null)
  // receive the activation memory before and after.  Tensors named in keep (a model's declared
  // outputs, which some operator may read as well) stay out of the plan.
  MaceStatus PlanMemory(size_t *separate_bytes, size_t *shared_bytes, const std::set<std::string> *keep = nullptr);
  bool captured() const { return graph_ != nullptr; }
  // Records `event` on the runtime's stream right after the last operator that reads the tensor
  // `input_name` (a net input), in every later Run(): the caller may refill that tensor for the
  // next run as soon as the event has happened, while the rest of the net still runs.  A
  // captured net is split into two graphs at that operator (the event is an ordinary stream
  // event between two graph launches).  event == nullptr takes the watch away.
  MaceStatus WatchInput(const std::string &input_name, void *event);
  // The next Run() makes the stream wait for `event` right behind the watch point (or at its
  // start when no input is watched): for a caller whose copy of the previous run's output must
  // be over before this run's later operators overwrite that tensor.  One-shot; nullptr = none.
  void WaitBehindWatchPoint(void *event) { wait_event_ = event; }
  ~SerialNet();
  size_t size() const { return operators_.size(); }

 private:
  const OpRegistry *op_registry_;
  Workspace *ws_;
  CudaRuntime *runtime_;
  std::vector<std::unique_ptr<OperatorDef>> defs_;
  std::vector<std::unique_ptr<Operation>> operators_;
  std::vector<char> skipped_;  // operators merged into their producer
  std::vector<void *> shared_buffers_;  // activation memory handed out by PlanMemory
  void *graph_ = nullptr;
  void *graph_tail_ = nullptr;   // the operators behind watch_index_ when an input is watched
  int watch_index_ = -1;         // last operator that reads the watched input
  void *watch_event_ = nullptr;
  void *wait_event_ = nullptr;   // one-shot: see WaitBehindWatchPoint
};

}  // namespace mace

#endif  // MACE_B200_HOST_OPS_H_
