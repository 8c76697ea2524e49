#include "mace_engine.h"

#include <algorithm>
#include <cstring>
#include <set>

namespace mace {

namespace {

size_t ProtoTypeSize(int data_type) {
  switch (data_type) {
    case 1: return 4;   // DT_FLOAT
    case 2: return 1;   // DT_UINT8
    case 3: return 2;   // DT_HALF
    case 4: return 4;   // DT_INT32
    case 5: return 2;   // DT_FLOAT16
    default: return 0;
  }
}

MaceStatus Invalid(const std::string &msg) { return MaceStatus(MaceStatus::MACE_INVALID_ARGS, msg); }

std::string Keys(const std::map<std::string, proto::InputOutputInfo> &m) {
  std::string s = "[";
  for (const auto &kv : m) s += (s.size() > 1 ? ", " : "") + kv.first;
  return s + "]";
}

}  // namespace

MaceEngine::~MaceEngine() {
  if (runtime_.ctx() != nullptr) {
    mb_stream_sync(runtime_.ctx());
    if (staging_ != nullptr) runtime_.Delete(staging_);
  }
}

MaceStatus MaceEngine::Staging(size_t bytes, void **ptr) {
  if (bytes > staging_bytes_) {
    // work queued on the old buffer ends before it is freed
    MACE_RETURN_IF_ERROR(runtime_.Status(mb_stream_sync(runtime_.ctx())));
    if (staging_ != nullptr) runtime_.Delete(staging_);
    staging_ = nullptr;
    staging_bytes_ = 0;
    MACE_RETURN_IF_ERROR(runtime_.New(bytes, &staging_));
    staging_bytes_ = bytes;
  }
  *ptr = staging_;
  return MaceStatus::MACE_SUCCESS;
}

MaceStatus MaceEngine::LoadModelTensors(const unsigned char *model_data, int64_t model_data_size) {
  if (net_def_.tensors.empty()) return MaceStatus::MACE_SUCCESS;
  if (model_data == nullptr || model_data_size <= 0)
    return Invalid("the model has constant tensors but no weights data was given");
  std::vector<float> widened;
  for (const proto::ConstTensor &ct : net_def_.tensors) {
    const size_t elem = ProtoTypeSize(ct.data_type);
    if (elem == 0) return MaceStatus(MaceStatus::MACE_UNSUPPORTED, "tensor " + ct.name + ": data type not supported");
    std::vector<index_t> dims(ct.dims.begin(), ct.dims.end());
    index_t count = 1;
    for (index_t d : dims) {
      if (d < 0) return Invalid("tensor " + ct.name + ": negative dimension");
      // (sizes come from a file: no product may leave the range of the blob's size)
      if (d != 0 && count > model_data_size / d) return Invalid("tensor " + ct.name + ": larger than the weights data");
      count *= d;
    }
    if (ct.offset < 0 || ct.data_size < 0) return Invalid("tensor " + ct.name + ": negative offset or size");
    if (count != ct.data_size) return Invalid("tensor " + ct.name + ": data_size not equal with the shape");
    if (ct.offset > model_data_size) return Invalid("tensor " + ct.name + ": offset beyond the weights data");
    const int64_t tensor_end = ct.offset + count * static_cast<int64_t>(elem);
    if (tensor_end > model_data_size)
      return Invalid("tensor " + ct.name + ": tensor_end (" + std::to_string(tensor_end) + ") should <= " +
                     std::to_string(model_data_size));
    const unsigned char *src = model_data + ct.offset;
    const bool half = ct.data_type == 3 || ct.data_type == 5;
    const bool dequantize = !quantized_ && ct.quantized;  // uint8-compressed weights of a float model
    const DataType dst_type = (half || dequantize) ? DT_FLOAT : static_cast<DataType>(ct.data_type);
    Tensor *t = workspace_.CreateTensor(ct.name, &runtime_, dst_type, true);
    MACE_RETURN_IF_ERROR(t->Resize(dims));
    t->SetScale(ct.scale);
    t->SetZeroPoint(ct.zero_point);
    if (count == 0) continue;
    const void *host = src;
    if (ct.data_type == 3) {
      widened.resize(static_cast<size_t>(count));
      for (index_t i = 0; i < count; ++i) {
        uint16_t h;
        std::memcpy(&h, src + 2 * i, 2);
        widened[static_cast<size_t>(i)] = HalfToFloat(h);
      }
      host = widened.data();
    } else if (ct.data_type == 5) {
      return MaceStatus(MaceStatus::MACE_UNSUPPORTED, "tensor " + ct.name + ": DT_FLOAT16 weights are not supported");
    } else if (dequantize) {
      if (ct.data_type != 2) return Invalid("tensor " + ct.name + ": quantized weights must be uint8");
      // QuantizeUtil::Dequantize (mace/core/quantize.h:184-194): scale * (q - zero_point)
      widened.resize(static_cast<size_t>(count));
      for (index_t i = 0; i < count; ++i)
        widened[static_cast<size_t>(i)] = ct.scale * static_cast<float>(static_cast<int>(src[i]) - ct.zero_point);
      host = widened.data();
    }
    MACE_RETURN_IF_ERROR(runtime_.Status(
        mb_memcpy_h2d(runtime_.ctx(), t->mutable_memory<void>(), host, static_cast<size_t>(t->raw_size()))));
    // the host copy (widened, or the caller's blob) may go away after Init
    MACE_RETURN_IF_ERROR(runtime_.Status(mb_stream_sync(runtime_.ctx())));
  }
  return MaceStatus::MACE_SUCCESS;
}

MaceStatus MaceEngine::Init(const proto::NetDef *net_def, const std::vector<std::string> &input_nodes,
                            const std::vector<std::string> &output_nodes, const unsigned char *model_data,
                            int64_t model_data_size) {
  if (net_def == nullptr) return Invalid("null NetDef");
  if (initialised_) return Invalid("the engine is initialised already");
  net_def_ = *net_def;
  quantized_ = GetNetArgInt(net_def_, "quantize_flag", 0) == 1;  // NetDefHelper::IsQuantizedModel
  for (const proto::InputOutputInfo &info : net_def_.input_info) input_info_[info.name] = info;
  for (const proto::InputOutputInfo &info : net_def_.output_info) output_info_[info.name] = info;
  for (const std::string &name : input_nodes)
    if (input_info_.count(name) == 0)
      return Invalid("'" + name + "' does not belong to model's inputs: " + Keys(input_info_));
  for (const std::string &name : output_nodes)
    if (output_info_.count(name) == 0)
      return Invalid("'" + name + "' does not belong to model's outputs: " + Keys(output_info_));

  if (config_.runtime_type() != RuntimeType::RT_CUDA)
    return MaceStatus(MaceStatus::MACE_UNSUPPORTED, "this engine runs RuntimeType::RT_CUDA only (no fallback)");
  MACE_RETURN_IF_ERROR(runtime_.Init(config_.device()));
  ops::RegisterAllCudaOpDelegators(workspace_.GetDelegatorRegistry());
  ops::RegisterAllCudaOps(&op_registry_);
  net_ = std::make_unique<SerialNet>(&op_registry_, &workspace_, &runtime_);

  MACE_RETURN_IF_ERROR(LoadModelTensors(model_data, model_data_size));

  for (const auto &kv : input_info_) {
    const proto::InputOutputInfo &info = kv.second;
    const DataType dt = static_cast<DataType>(info.data_type);
    if (GetEnumTypeSize(dt) == 0) return MaceStatus(MaceStatus::MACE_UNSUPPORTED, "input " + info.name + ": data type");
    std::vector<index_t> shape(info.dims.begin(), info.dims.end());
    // the file states the shape in the layout named by data_format; a float model runs NCHW
    if (!quantized_ && shape.size() == 4 && info.data_format == static_cast<int>(DataFormat::NHWC))
      shape = {shape[0], shape[3], shape[1], shape[2]};
    else if (quantized_ && shape.size() == 4 && info.data_format == static_cast<int>(DataFormat::NCHW))
      shape = {shape[0], shape[2], shape[3], shape[1]};
    Tensor *t = workspace_.CreateTensor(info.name, &runtime_, dt, false);
    MACE_RETURN_IF_ERROR(t->Resize(shape));
    t->SetScale(info.scale);
    t->SetZeroPoint(info.zero_point);
  }

  for (const proto::OperatorDef &op : net_def_.op) {
    OperatorDef def;
    ConvertOperatorDef(op, &def);
    MaceStatus st = net_->AddOperator(def);
    if (st != MaceStatus::MACE_SUCCESS)
      return MaceStatus(st.code(), "operator " + op.name + " (" + op.type + "): " + st.information());
  }
  for (const auto &kv : output_info_)
    if (!workspace_.HasTensor(kv.first)) return Invalid("no operator produces the model output " + kv.first);
  if (config_.fuse()) net_->ShareSubsampledInputs();
  initialised_ = true;
  return MaceStatus::MACE_SUCCESS;
}

MaceStatus MaceEngine::Run(const std::map<std::string, MaceTensor> &inputs, std::map<std::string, MaceTensor> *outputs,
                           RunMetadata *run_metadata) {
  if (!initialised_) return Invalid("the engine is not initialised");
  if (outputs == nullptr) return Invalid("null outputs");
  mb_context *ctx = runtime_.ctx();

  // ---- inputs: host -> device, transposed to the layout the model runs in ----
  for (const auto &in : inputs) {
    auto info_it = input_info_.find(in.first);
    if (info_it == input_info_.end())
      return Invalid("'" + in.first + "' does not belong to model's inputs: " + Keys(input_info_));
    const proto::InputOutputInfo &info = info_it->second;
    const MaceTensor &mt = in.second;
    Tensor *t = workspace_.GetTensor(in.first);
    if (mt.data_ == nullptr) return Invalid("input " + in.first + " has no data");
    if (static_cast<int>(mt.data_type_) != static_cast<int>(t->dtype()))
      return Invalid("input " + in.first + ": data type does not match the model's");
    std::vector<index_t> shape(mt.shape_.begin(), mt.shape_.end());
    for (index_t d : shape)
      if (d < 0) return Invalid("input " + in.first + ": negative dimension");
    bool to_nchw = false, to_nhwc = false;
    if (info.data_format != static_cast<int>(DataFormat::NONE) && shape.size() == 4) {
      to_nchw = !quantized_ && mt.format_ == DataFormat::NHWC;
      to_nhwc = quantized_ && mt.format_ == DataFormat::NCHW;
    }
    index_t rows = 0, cols = 0;
    if (to_nchw) {
      rows = shape[1] * shape[2];
      cols = shape[3];
      shape = {shape[0], shape[3], shape[1], shape[2]};
    } else if (to_nhwc) {
      rows = shape[1];
      cols = shape[2] * shape[3];
      shape = {shape[0], shape[2], shape[3], shape[1]};
    }
    if (shape != t->shape()) {
      net_->DropCapture();  // a recorded graph holds the old shapes and addresses
      plain_runs_ = 0;
      MACE_RETURN_IF_ERROR(t->Resize(shape));
    }
    const size_t bytes = static_cast<size_t>(t->raw_size());
    if (bytes == 0) continue;
    if (to_nchw || to_nhwc) {
      void *stage = nullptr;
      MACE_RETURN_IF_ERROR(Staging(bytes, &stage));
      MACE_RETURN_IF_ERROR(runtime_.Status(mb_memcpy_h2d(ctx, stage, mt.data_.get(), bytes)));
      MACE_RETURN_IF_ERROR(runtime_.Status(mb_transpose2d_batched(
          ctx, stage, t->mutable_memory<void>(), shape[0], rows, cols, static_cast<int>(GetEnumTypeSize(t->dtype())))));
    } else {
      MACE_RETURN_IF_ERROR(runtime_.Status(mb_memcpy_h2d(ctx, t->mutable_memory<void>(), mt.data_.get(), bytes)));
    }
  }
  for (const auto &out : *outputs)
    if (output_info_.count(out.first) == 0)
      return Invalid("'" + out.first + "' does not belong to model's outputs: " + Keys(output_info_));

  // ---- the net ----
  if (config_.cuda_graph() && !graph_failed_ && !net_->captured() && plain_runs_ >= 1 && run_metadata == nullptr) {
    if (net_->Capture() != MaceStatus::MACE_SUCCESS) graph_failed_ = true;  // an operator that must wait for the host
  }
  MACE_RETURN_IF_ERROR(net_->Run(run_metadata));
  if (!net_->captured()) ++plain_runs_;
  if (!optimised_) {
    optimised_ = true;
    // a declared output is always written, and keeps memory of its own even when another
    // operator reads it too, so that it can be read back after the run
    std::set<std::string> keep;
    for (const auto &kv : output_info_) keep.insert(kv.first);
    if (config_.fuse()) {
      net_->FuseActivations(&keep);
      net_->FuseResidualSums(&keep);
      plain_runs_ = 0;
    }
    if (config_.plan_memory()) {
      MACE_RETURN_IF_ERROR(net_->PlanMemory(nullptr, nullptr, &keep));
      plain_runs_ = 0;
    }
  }

  // ---- outputs: device -> host, transposed to the layout the caller asked for ----
  for (auto &out : *outputs) {
    const proto::InputOutputInfo &info = output_info_[out.first];
    MaceTensor &mt = out.second;
    const Tensor *t = workspace_.GetTensor(out.first);
    if (mt.data_ == nullptr) return Invalid("output " + out.first + " has no buffer");
    if (static_cast<int>(mt.data_type_) != static_cast<int>(t->dtype()))
      return Invalid("output " + out.first + ": data type does not match the model's");
    std::vector<index_t> shape = t->shape();
    // the layout the tensor has on the device: NCHW in a float model, NHWC in a quantized one
    const DataFormat have = info.data_format == static_cast<int>(DataFormat::NONE)
                                ? DataFormat::NONE
                                : (quantized_ ? DataFormat::NHWC : DataFormat::NCHW);
    index_t rows = 0, cols = 0;
    bool transpose = false;
    if (have != DataFormat::NONE && mt.format_ != DataFormat::NONE && shape.size() == 4 && mt.shape_.size() == 4 &&
        mt.format_ != have) {
      transpose = true;
      if (have == DataFormat::NCHW && mt.format_ == DataFormat::NHWC) {
        rows = shape[1];
        cols = shape[2] * shape[3];
        shape = {shape[0], shape[2], shape[3], shape[1]};
      } else if (have == DataFormat::NHWC && mt.format_ == DataFormat::NCHW) {
        rows = shape[1] * shape[2];
        cols = shape[3];
        shape = {shape[0], shape[3], shape[1], shape[2]};
      } else {
        return Invalid("Not supported output data format");
      }
    }
    if (t->size() > mt.buffer_size_)
      return Invalid("Output size exceeds buffer size: output " + out.first + " has " + std::to_string(t->size()) +
                     " elements, the buffer " + std::to_string(mt.buffer_size_));
    mt.shape_.assign(shape.begin(), shape.end());
    const size_t bytes = static_cast<size_t>(t->raw_size());
    if (bytes == 0) continue;
    if (transpose) {
      void *stage = nullptr;
      MACE_RETURN_IF_ERROR(Staging(bytes, &stage));
      MACE_RETURN_IF_ERROR(runtime_.Status(mb_transpose2d_batched(
          ctx, t->memory<void>(), stage, t->dim(0), rows, cols, static_cast<int>(GetEnumTypeSize(t->dtype())))));
      MACE_RETURN_IF_ERROR(runtime_.Status(mb_memcpy_d2h(ctx, mt.data_.get(), stage, bytes)));
      // the staging buffer is reused by the next output
      MACE_RETURN_IF_ERROR(runtime_.Status(mb_stream_sync(ctx)));
    } else {
      MACE_RETURN_IF_ERROR(runtime_.Status(mb_memcpy_d2h(ctx, mt.data_.get(), t->memory<void>(), bytes)));
    }
  }
  return runtime_.Status(mb_stream_sync(ctx));
}

MaceStatus CreateMaceEngineFromProto(const unsigned char *model_graph_proto, size_t model_graph_proto_size,
                                     const unsigned char *model_weights_data, size_t model_weights_data_size,
                                     const std::vector<std::string> &input_nodes,
                                     const std::vector<std::string> &output_nodes, const MaceEngineConfig &config,
                                     std::shared_ptr<MaceEngine> *engine, bool *model_data_unused,
                                     MaceEngine *tutor, bool fake_warmup) {
  (void)tutor;
  (void)fake_warmup;
  if (engine == nullptr) return Invalid("null engine pointer");
  if (model_graph_proto == nullptr || model_graph_proto_size == 0) return Invalid("empty model graph");
  proto::NetDef net_def;
  MACE_RETURN_IF_ERROR(ParseNetDef(model_graph_proto, model_graph_proto_size, &net_def));
  auto e = std::make_shared<MaceEngine>(config);
  MACE_RETURN_IF_ERROR(e->Init(&net_def, input_nodes, output_nodes, model_weights_data,
                               static_cast<int64_t>(model_weights_data_size)));
  *engine = std::move(e);
  if (model_data_unused != nullptr) *model_data_unused = true;
  return MaceStatus::MACE_SUCCESS;
}

}  // namespace mace
