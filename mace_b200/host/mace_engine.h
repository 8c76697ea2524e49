// The model-level API of MACE for the CUDA runtime: MaceTensor, MaceEngineConfig, MaceEngine
// and CreateMaceEngineFromProto with the meaning they have in include/mace/public/mace.h:500-660
// -- a converted model (the serialized NetDef plus its weights blob) is loaded and run on host
// buffers, unchanged.  What the CPU engine does at this level is restated here:
//   * constant tensors are cut out of the weights blob by offset and size; DT_HALF weights are
//     widened to float and uint8-compressed weights of a float model are dequantized
//     (Workspace::LoadModelTensor, mace/core/workspace.cc:102-176);
//   * input tensors are created from input_info (BaseFlow::InitInputTensors,
//     mace/core/flow/base_flow.cc:301-319);
//   * a float model runs NCHW, a quantized one NHWC: 4-D inputs and outputs handed over in the
//     other layout are transposed on the way in and out (CpuRefFlow::GetInputTransposeDims,
//     mace/flows/cpu/cpu_ref_flow.cc:81-101; BaseFlow::GetOutputTransposeDims,
//     mace/core/flow/base_flow.cc:131-208, BaseFlow::Run, :75-116) -- on the device here;
//   * the operators run in file order (SerialNet::Run, mace/core/net/serial_net.cc:103-124).
// Not restated: MultiNetDef, model files read from disk, OpenCL/Hexagon/APU options.
#ifndef MACE_B200_HOST_MACE_ENGINE_H_
#define MACE_B200_HOST_MACE_ENGINE_H_

#include <map>
#include <memory>
#include <string>
#include <vector>

#include "netdef.h"
#include "ops.h"

namespace mace {

enum IDataType {  // include/mace/public/mace.h:64-76, the same values as DataType
  IDT_INVALID = 0,
  IDT_FLOAT = 1,
  IDT_UINT8 = 2,
  IDT_HALF = 3,
  IDT_INT32 = 4,
};

// An input or output in HOST memory (include/mace/public/mace.h:501-551).
class MaceTensor {
 public:
  MaceTensor() = default;
  MaceTensor(const std::vector<int64_t> &shape, std::shared_ptr<void> data,
             const DataFormat format = DataFormat::NHWC, const IDataType data_type = IDT_FLOAT)
      : shape_(shape), data_(std::move(data)), format_(format), data_type_(data_type) {
    buffer_size_ = 1;
    for (int64_t d : shape_) buffer_size_ *= d;
  }
  // After a run: the actual shape of an output.
  const std::vector<int64_t> &shape() const { return shape_; }
  template <typename T> std::shared_ptr<T> data() const { return std::static_pointer_cast<T>(data_); }
  DataFormat data_format() const { return format_; }
  IDataType data_type() const { return data_type_; }
  // Elements the buffer holds (the product of the shape it was constructed with).
  int64_t buffer_size() const { return buffer_size_; }

 private:
  friend class MaceEngine;
  std::vector<int64_t> shape_;
  std::shared_ptr<void> data_;
  DataFormat format_ = DataFormat::NHWC;
  IDataType data_type_ = IDT_FLOAT;
  int64_t buffer_size_ = 0;
};

// Hints of the reference's configuration class that this runtime accepts and ignores
// (include/mace/public/mace.h:91-143): they steer CPU threads and mobile GPUs.
enum GPUPerfHint { PERF_DEFAULT = 0, PERF_LOW = 1, PERF_NORMAL = 2, PERF_HIGH = 3 };
enum GPUPriorityHint { PRIORITY_DEFAULT = 0, PRIORITY_LOW = 1, PRIORITY_NORMAL = 2, PRIORITY_HIGH = 3 };
enum CPUAffinityPolicy {
  AFFINITY_NONE = 0, AFFINITY_BIG_ONLY = 1, AFFINITY_LITTLE_ONLY = 2, AFFINITY_HIGH_PERFORMANCE = 3,
  AFFINITY_POWER_SAVE = 4,
};

// The setters of include/mace/public/mace.h:372-499 that have a meaning for one CUDA device,
// with the same names and return types, so that code configuring a MACE engine compiles against
// this runtime: SetRuntimeType takes RT_CUDA (any other runtime makes Init fail with
// MACE_UNSUPPORTED, there is no fallback), the CPU and GPU hints are accepted and have no
// effect.  Additions for this runtime: the device ordinal and the three net-level switches.
// Unlike the reference's class this one can be copied (one configuration for several engines).
class MaceEngineConfig {
 public:
  MaceEngineConfig() = default;
  explicit MaceEngineConfig(const RuntimeType runtime_type) : runtime_type_(runtime_type) {}

  void SetRuntimeType(const RuntimeType runtime_type, const char *sub_graph_name = "default_graph") {
    (void)sub_graph_name;  // one graph per model file
    runtime_type_ = runtime_type;
  }
  MaceStatus SetGPUHints(GPUPerfHint perf_hint, GPUPriorityHint priority_hint) {
    (void)perf_hint;
    (void)priority_hint;
    return MaceStatus::MACE_SUCCESS;
  }
  MaceStatus SetCPUThreadPolicy(int num_threads_hint, CPUAffinityPolicy policy) {
    (void)num_threads_hint;
    (void)policy;
    return MaceStatus::MACE_SUCCESS;
  }
  // ---- this runtime ----
  MaceStatus SetCudaDevice(int ordinal) {
    if (ordinal < 0) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "negative device ordinal");
    device_ = ordinal;
    return MaceStatus::MACE_SUCCESS;
  }
  // After the first run: merge activations and residual sums into their producers
  // (SerialNet::FuseActivations / FuseResidualSums), share activation memory
  // (SerialNet::PlanMemory), and record the operator chain into a CUDA graph that later runs
  // with unchanged input shapes replay.
  MaceStatus SetCudaNetOptimizations(bool fuse, bool plan_memory, bool cuda_graph) {
    fuse_ = fuse;
    plan_memory_ = plan_memory;
    cuda_graph_ = cuda_graph;
    return MaceStatus::MACE_SUCCESS;
  }
  RuntimeType runtime_type() const { return runtime_type_; }
  int device() const { return device_; }
  bool fuse() const { return fuse_; }
  bool plan_memory() const { return plan_memory_; }
  bool cuda_graph() const { return cuda_graph_; }

 private:
  RuntimeType runtime_type_ = RuntimeType::RT_CUDA;
  int device_ = 0;
  bool fuse_ = false;
  bool plan_memory_ = false;
  bool cuda_graph_ = false;
};

class MaceEngine {
 public:
  explicit MaceEngine(const MaceEngineConfig &config) : config_(config) {}
  ~MaceEngine();
  MaceEngine(const MaceEngine &) = delete;
  MaceEngine &operator=(const MaceEngine &) = delete;

  // input_nodes / output_nodes must be names of the model's input_info / output_info
  // (MACE_INVALID_ARGS otherwise); model_data may be null for a model without weights.
  MaceStatus Init(const proto::NetDef *net_def, const std::vector<std::string> &input_nodes,
                  const std::vector<std::string> &output_nodes, const unsigned char *model_data,
                  int64_t model_data_size);
  // include/mace/public/mace.h:603-607; run_metadata (may be null) receives one OperatorStats per
  // operator, timed with device events.
  MaceStatus Run(const std::map<std::string, MaceTensor> &inputs, std::map<std::string, MaceTensor> *outputs,
                 RunMetadata *run_metadata = nullptr);

  const proto::NetDef &net_def() const { return net_def_; }
  bool is_quantized_model() const { return quantized_; }
  CudaRuntime *runtime() { return &runtime_; }
  SerialNet *net() { return net_.get(); }
  Workspace *workspace() { return &workspace_; }

 private:
  MaceStatus LoadModelTensors(const unsigned char *model_data, int64_t model_data_size);
  MaceStatus Staging(size_t bytes, void **ptr);

  MaceEngineConfig config_;
  proto::NetDef net_def_;
  bool quantized_ = false;
  bool initialised_ = false;
  CudaRuntime runtime_;
  Workspace workspace_;
  OpRegistry op_registry_;
  std::unique_ptr<SerialNet> net_;
  std::map<std::string, proto::InputOutputInfo> input_info_, output_info_;
  int plain_runs_ = 0;  // runs outside a graph since the last change of shapes or operators
  bool graph_failed_ = false;
  bool optimised_ = false;
  void *staging_ = nullptr;
  size_t staging_bytes_ = 0;
};

// include/mace/public/mace.h:644-655: parses the graph, builds and initialises an engine.
// *model_data_unused (may be null) is set to true: every constant tensor is copied to the device
// during Init, so the caller may release the weights blob.  tutor (an engine whose runtimes the
// new one would share) and fake_warmup (an OpenCL start-up aid) are accepted and have no effect:
// every engine of this runtime owns its stream and memory.
MaceStatus CreateMaceEngineFromProto(const unsigned char *model_graph_proto, size_t model_graph_proto_size,
                                     const unsigned char *model_weights_data, size_t model_weights_data_size,
                                     const std::vector<std::string> &input_nodes,
                                     const std::vector<std::string> &output_nodes, const MaceEngineConfig &config,
                                     std::shared_ptr<MaceEngine> *engine, bool *model_data_unused = nullptr,
                                     MaceEngine *tutor = nullptr, bool fake_warmup = false);

}  // namespace mace

#endif  // MACE_B200_HOST_MACE_ENGINE_H_
