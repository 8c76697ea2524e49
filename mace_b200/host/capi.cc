#include "capi.h"

#include <algorithm>
#include <cstring>
#include <exception>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "logging.h"
#include "mace_engine.h"
#include "multi_gpu.h"
#include "ops.h"

using namespace mace;  // NOLINT

struct mbh_engine {
  CudaRuntime runtime;
  Workspace workspace;
  OpRegistry op_registry;
  std::unique_ptr<SerialNet> net;
  OperatorDef pending;
  bool building = false;
  std::string last_error;
  // mbh_run_host_pipelined: an event "the net has read its input" and, per slot, an event
  // "output in host memory"
  void *consumed = nullptr;
  std::string watched_input;
  void *done[2] = {nullptr, nullptr};
  uint64_t pipelined_calls = 0;
};

namespace {

int Fail(mbh_engine *e, const MaceStatus &st) {
  if (e != nullptr) e->last_error = st.information();
  return static_cast<int>(st.code());
}

int Fail(mbh_engine *e, MaceStatus::Code code, const std::string &msg) {
  if (e != nullptr) e->last_error = msg;
  return static_cast<int>(code);
}

#define MBH_TRY(e, expr)                                             \
  do {                                                               \
    MaceStatus _st = (expr);                                         \
    if (_st != MaceStatus::MACE_SUCCESS) return Fail((e), _st);      \
  } while (0)

}  // namespace

extern "C" {

int mbh_engine_create(int device, mbh_engine **engine) {
  if (engine == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  *engine = nullptr;
  mbh_engine *e = new mbh_engine();
  MaceStatus st = e->runtime.Init(device);
  if (st != MaceStatus::MACE_SUCCESS) {
    const int rc = static_cast<int>(st.code());
    delete e;
    return rc;
  }
  ops::RegisterAllCudaOpDelegators(e->workspace.GetDelegatorRegistry());
  ops::RegisterAllCudaOps(&e->op_registry);
  e->net = std::make_unique<SerialNet>(&e->op_registry, &e->workspace, &e->runtime);
  *engine = e;
  return MaceStatus::MACE_SUCCESS;
}

int mbh_engine_destroy(mbh_engine *engine) {
  if (engine == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  mb_stream_sync(engine->runtime.ctx());
  if (engine->consumed != nullptr) mb_event_destroy(engine->runtime.ctx(), engine->consumed);
  for (int i = 0; i < 2; ++i)
    if (engine->done[i] != nullptr) mb_event_destroy(engine->runtime.ctx(), engine->done[i]);
  delete engine;
  return MaceStatus::MACE_SUCCESS;
}

const char *mbh_last_error(const mbh_engine *engine) {
  return engine ? engine->last_error.c_str() : "null engine";
}

void *mbh_engine_context(mbh_engine *engine) { return engine ? engine->runtime.ctx() : nullptr; }

int mbh_add_tensor(mbh_engine *e, const char *name, int data_type, int rank, const int64_t *dims,
                   const void *host_data, float scale, int32_t zero_point, int is_weight) {
  if (e == nullptr || name == nullptr || rank < 0 || (rank > 0 && dims == nullptr))
    return MaceStatus::MACE_INVALID_ARGS;
  const DataType dt = static_cast<DataType>(data_type);
  if (GetEnumTypeSize(dt) == 0) return Fail(e, MaceStatus::MACE_INVALID_ARGS, "unsupported data type");
  std::vector<index_t> shape(dims, dims + rank);
  for (index_t d : shape)
    if (d < 0) return Fail(e, MaceStatus::MACE_INVALID_ARGS, "negative dimension");
  e->net->DropCapture();  // a recorded graph holds the old tensor's address
  Tensor *t = e->workspace.CreateTensor(name, &e->runtime, dt, is_weight != 0);
  MBH_TRY(e, t->Resize(shape));
  t->SetScale(scale);
  t->SetZeroPoint(zero_point);
  if (host_data != nullptr && t->raw_size() > 0) {
    MBH_TRY(e, e->runtime.Status(mb_memcpy_h2d(e->runtime.ctx(), t->mutable_memory<void>(), host_data,
                                               static_cast<size_t>(t->raw_size()))));
    MBH_TRY(e, e->runtime.Status(mb_stream_sync(e->runtime.ctx())));
  }
  return MaceStatus::MACE_SUCCESS;
}

static Tensor *FindTensor(mbh_engine *e, const char *name) {
  if (e == nullptr || name == nullptr) return nullptr;
  Tensor *t = e->workspace.GetTensor(name);
  if (t == nullptr) e->last_error = std::string("no tensor named ") + name;
  return t;
}

int mbh_set_tensor_quant(mbh_engine *e, const char *name, float scale, int32_t zero_point) {
  Tensor *t = FindTensor(e, name);
  if (t == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  t->SetScale(scale);
  t->SetZeroPoint(zero_point);
  return MaceStatus::MACE_SUCCESS;
}

int mbh_tensor_rank(mbh_engine *e, const char *name, int *rank) {
  Tensor *t = FindTensor(e, name);
  if (t == nullptr || rank == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  *rank = static_cast<int>(t->dim_size());
  return MaceStatus::MACE_SUCCESS;
}

int mbh_tensor_shape(mbh_engine *e, const char *name, int64_t *dims, int max_rank) {
  Tensor *t = FindTensor(e, name);
  if (t == nullptr || dims == nullptr || max_rank < t->dim_size()) return MaceStatus::MACE_INVALID_ARGS;
  for (index_t i = 0; i < t->dim_size(); ++i) dims[i] = t->dim(static_cast<unsigned>(i));
  return MaceStatus::MACE_SUCCESS;
}

int mbh_tensor_quant(mbh_engine *e, const char *name, float *scale, int32_t *zero_point) {
  Tensor *t = FindTensor(e, name);
  if (t == nullptr || scale == nullptr || zero_point == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  *scale = t->scale();
  *zero_point = t->zero_point();
  return MaceStatus::MACE_SUCCESS;
}

int mbh_tensor_read(mbh_engine *e, const char *name, void *host_out, size_t bytes) {
  Tensor *t = FindTensor(e, name);
  if (t == nullptr || (bytes != 0 && host_out == nullptr)) return MaceStatus::MACE_INVALID_ARGS;
  if (bytes > static_cast<size_t>(t->raw_size()))
    return Fail(e, MaceStatus::MACE_INVALID_ARGS, "read larger than the tensor");
  MBH_TRY(e, e->runtime.Status(mb_memcpy_d2h(e->runtime.ctx(), host_out, t->memory<void>(), bytes)));
  MBH_TRY(e, e->runtime.Status(mb_stream_sync(e->runtime.ctx())));
  return MaceStatus::MACE_SUCCESS;
}

int mbh_tensor_device_ptr(mbh_engine *e, const char *name, void **device_ptr, size_t *bytes) {
  Tensor *t = FindTensor(e, name);
  if (t == nullptr || device_ptr == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  *device_ptr = t->mutable_memory<void>();
  if (bytes != nullptr) *bytes = static_cast<size_t>(t->raw_size());
  return MaceStatus::MACE_SUCCESS;
}

int mbh_tensor_write(mbh_engine *e, const char *name, const void *host_in, size_t bytes) {
  Tensor *t = FindTensor(e, name);
  if (t == nullptr || (bytes != 0 && host_in == nullptr)) return MaceStatus::MACE_INVALID_ARGS;
  if (bytes > static_cast<size_t>(t->raw_size()))
    return Fail(e, MaceStatus::MACE_INVALID_ARGS, "write larger than the tensor");
  MBH_TRY(e, e->runtime.Status(mb_memcpy_h2d(e->runtime.ctx(), t->mutable_memory<void>(), host_in, bytes)));
  MBH_TRY(e, e->runtime.Status(mb_stream_sync(e->runtime.ctx())));
  return MaceStatus::MACE_SUCCESS;
}

int mbh_op_begin(mbh_engine *e, const char *type, const char *name) {
  if (e == nullptr || type == nullptr || name == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  e->pending = OperatorDef();
  e->pending.type = type;
  e->pending.name = name;
  e->building = true;
  return MaceStatus::MACE_SUCCESS;
}

int mbh_op_input(mbh_engine *e, const char *tensor_name) {
  if (e == nullptr || !e->building || tensor_name == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  e->pending.input.push_back(tensor_name);
  return MaceStatus::MACE_SUCCESS;
}

int mbh_op_output(mbh_engine *e, const char *tensor_name, int data_type, float scale, int32_t zero_point) {
  if (e == nullptr || !e->building || tensor_name == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  e->pending.output.push_back(tensor_name);
  if (data_type >= 0) {
    e->pending.output_type.resize(e->pending.output.size(), DT_INVALID);
    e->pending.output_type.back() = static_cast<DataType>(data_type);
  }
  if (scale > 0.f) {
    e->pending.quantize_info.resize(e->pending.output.size());
    e->pending.quantize_info.back().scale = scale;
    e->pending.quantize_info.back().zero_point = zero_point;
  }
  return MaceStatus::MACE_SUCCESS;
}

int mbh_op_arg_int(mbh_engine *e, const char *key, int value) {
  if (e == nullptr || !e->building || key == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  e->pending.i[key] = value;
  return MaceStatus::MACE_SUCCESS;
}

int mbh_op_arg_ints(mbh_engine *e, const char *key, int count, const int *values) {
  if (e == nullptr || !e->building || key == nullptr || count < 0 || (count > 0 && values == nullptr))
    return MaceStatus::MACE_INVALID_ARGS;
  e->pending.ints[key] = std::vector<int>(values, values + count);
  return MaceStatus::MACE_SUCCESS;
}

int mbh_op_arg_floats(mbh_engine *e, const char *key, int count, const float *values) {
  if (e == nullptr || !e->building || key == nullptr || count < 0 || (count > 0 && values == nullptr))
    return MaceStatus::MACE_INVALID_ARGS;
  e->pending.floats[key] = std::vector<float>(values, values + count);
  return MaceStatus::MACE_SUCCESS;
}

int mbh_op_arg_float(mbh_engine *e, const char *key, float value) {
  if (e == nullptr || !e->building || key == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  e->pending.f[key] = value;
  return MaceStatus::MACE_SUCCESS;
}

int mbh_op_arg_str(mbh_engine *e, const char *key, const char *value) {
  if (e == nullptr || !e->building || key == nullptr || value == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  e->pending.s[key] = value;
  return MaceStatus::MACE_SUCCESS;
}

int mbh_op_end(mbh_engine *e) {
  if (e == nullptr || !e->building) return MaceStatus::MACE_INVALID_ARGS;
  e->building = false;
  // an output_type entry left DT_INVALID means "use T"
  for (auto &dt : e->pending.output_type) {
    if (dt == DT_INVALID) {
      auto it = e->pending.i.find("T");
      dt = it == e->pending.i.end() ? DT_FLOAT : static_cast<DataType>(it->second);
    }
  }
  MBH_TRY(e, e->net->AddOperator(e->pending));
  return MaceStatus::MACE_SUCCESS;
}

// A run that is not part of the pipelined sequence must not overwrite the output tensor while the
// last pipelined call's copy to the host may still read it.
static void WaitForLastDownload(mbh_engine *e) {
  if (e->pipelined_calls >= 1) e->net->WaitBehindWatchPoint(e->done[(e->pipelined_calls - 1) & 1]);
}

int mbh_run(mbh_engine *e) {
  if (e == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  WaitForLastDownload(e);
  MBH_TRY(e, e->net->Run(nullptr));
  return MaceStatus::MACE_SUCCESS;
}

int mbh_fuse_activations(mbh_engine *e, int *merged) {
  if (e == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  const int n = e->net->FuseActivations();
  if (merged != nullptr) *merged = n;
  return MaceStatus::MACE_SUCCESS;
}

int mbh_fuse_residual_sums(mbh_engine *e, int *merged) {
  if (e == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  const int n = e->net->FuseResidualSums();
  if (merged != nullptr) *merged = n;
  return MaceStatus::MACE_SUCCESS;
}

int mbh_share_subsampled_inputs(mbh_engine *e, int *groups) {
  if (e == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  const int n = e->net->ShareSubsampledInputs();
  if (groups != nullptr) *groups = n;
  return MaceStatus::MACE_SUCCESS;
}

int mbh_plan_memory(mbh_engine *e, size_t *separate_bytes, size_t *shared_bytes) {
  if (e == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  MBH_TRY(e, e->net->PlanMemory(separate_bytes, shared_bytes));
  return MaceStatus::MACE_SUCCESS;
}

int mbh_capture(mbh_engine *e) {
  if (e == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  MBH_TRY(e, e->net->Capture());
  return MaceStatus::MACE_SUCCESS;
}

int mbh_sync(mbh_engine *e) {
  if (e == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  MBH_TRY(e, e->runtime.Status(mb_stream_sync(e->runtime.ctx())));
  return MaceStatus::MACE_SUCCESS;
}

int mbh_run_host(mbh_engine *e, const char *input_name, const void *host_in, size_t input_bytes,
                 const char *output_name, void *host_out, size_t output_bytes) {
  Tensor *in = FindTensor(e, input_name);
  if (in == nullptr || host_in == nullptr || host_out == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  if (input_bytes != static_cast<size_t>(in->raw_size()))
    return Fail(e, MaceStatus::MACE_INVALID_ARGS, "input size does not match the input tensor");
  MBH_TRY(e, e->runtime.Status(mb_memcpy_h2d(e->runtime.ctx(), in->mutable_memory<void>(), host_in, input_bytes)));
  WaitForLastDownload(e);
  MBH_TRY(e, e->net->Run(nullptr));
  Tensor *out = FindTensor(e, output_name);
  if (out == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  if (output_bytes != static_cast<size_t>(out->raw_size()))
    return Fail(e, MaceStatus::MACE_INVALID_ARGS, "output size does not match the output tensor");
  MBH_TRY(e, e->runtime.Status(mb_memcpy_d2h(e->runtime.ctx(), host_out, out->memory<void>(), output_bytes)));
  MBH_TRY(e, e->runtime.Status(mb_stream_sync(e->runtime.ctx())));
  return MaceStatus::MACE_SUCCESS;
}

int mbh_run_host_pipelined(mbh_engine *e, const char *input_name, const void *host_in, size_t input_bytes,
                           const char *output_name, void *host_out, size_t output_bytes, int *slot_out) {
  Tensor *in = FindTensor(e, input_name);
  Tensor *out = FindTensor(e, output_name);
  if (in == nullptr || out == nullptr || host_in == nullptr || host_out == nullptr)
    return MaceStatus::MACE_INVALID_ARGS;
  if (input_bytes != static_cast<size_t>(in->raw_size()))
    return Fail(e, MaceStatus::MACE_INVALID_ARGS, "input size does not match the input tensor");
  if (output_bytes != static_cast<size_t>(out->raw_size()))
    return Fail(e, MaceStatus::MACE_INVALID_ARGS, "output size does not match the output tensor (run the net once first)");
  mb_context *ctx = e->runtime.ctx();
  for (int i = 0; i < 2; ++i)
    if (e->done[i] == nullptr) MBH_TRY(e, e->runtime.Status(mb_event_create(ctx, &e->done[i])));
  if (e->consumed == nullptr) MBH_TRY(e, e->runtime.Status(mb_event_create(ctx, &e->consumed)));
  // The net records `consumed` behind the last operator that reads the input tensor (a captured
  // net is two graphs with the event between them), so the upload of the NEXT call goes
  // straight into the input tensor as soon as this call's first operators are through, while
  // the rest of the net still runs: no staging copy inside device memory.
  if (e->watched_input != input_name) {
    MBH_TRY(e, e->net->WatchInput(input_name, e->consumed));
    e->watched_input = input_name;
    e->pipelined_calls = 0;
  }
  const int slot = static_cast<int>(e->pipelined_calls & 1);
  if (e->pipelined_calls >= 1) MBH_TRY(e, e->runtime.Status(mb_upload_wait_event(ctx, e->consumed)));
  MBH_TRY(e, e->runtime.Status(mb_upload_h2d(ctx, in->mutable_memory<void>(), host_in, input_bytes)));
  MBH_TRY(e, e->runtime.Status(mb_upload_signal(ctx)));
  // The copy of the output to the host runs on its own stream, so the next call's first
  // operators do not queue behind it; that call's net waits for it behind its watch point, before
  // any later operator can overwrite the output tensor.
  if (e->pipelined_calls >= 1) e->net->WaitBehindWatchPoint(e->done[slot ^ 1]);
  MBH_TRY(e, e->net->Run(nullptr));
  MBH_TRY(e, e->runtime.Status(mb_download_d2h(ctx, host_out, out->memory<void>(), output_bytes, e->done[slot])));
  e->pipelined_calls++;
  if (slot_out != nullptr) *slot_out = slot;
  return MaceStatus::MACE_SUCCESS;
}

int mbh_wait_slot(mbh_engine *e, int slot) {
  if (e == nullptr || slot < 0 || slot > 1 || e->done[slot] == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  MBH_TRY(e, e->runtime.Status(mb_event_sync(e->runtime.ctx(), e->done[slot])));
  return MaceStatus::MACE_SUCCESS;
}

int mbh_run_profiled(mbh_engine *e, float *ms_out, int max_ops, char *names_out, size_t names_len,
                     int *op_count) {
  if (e == nullptr || ms_out == nullptr || op_count == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  RunMetadata metadata;
  MBH_TRY(e, e->net->Run(&metadata));
  const std::vector<OperatorStats> &stats = metadata.op_stats;
  *op_count = static_cast<int>(stats.size());
  std::string names;
  for (size_t i = 0; i < stats.size(); ++i) {
    if (static_cast<int>(i) < max_ops) ms_out[i] = stats[i].device_ms;
    names += stats[i].type + ":" + stats[i].operator_name + "\n";
  }
  if (names_out != nullptr && names_len > 0) {
    std::strncpy(names_out, names.c_str(), names_len - 1);
    names_out[names_len - 1] = 0;
  }
  return MaceStatus::MACE_SUCCESS;
}

int mbh_run_profiled_graph(mbh_engine *e, int replays, float *ms_out, int max_ops, char *names_out,
                           size_t names_len, int *op_count) {
  if (e == nullptr || ms_out == nullptr || op_count == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  RunMetadata metadata;
  MBH_TRY(e, e->net->RunProfiledGraph(&metadata, replays));
  const std::vector<OperatorStats> &stats = metadata.op_stats;
  *op_count = static_cast<int>(stats.size());
  std::string names;
  for (size_t i = 0; i < stats.size(); ++i) {
    if (static_cast<int>(i) < max_ops) ms_out[i] = stats[i].device_ms;
    names += stats[i].type + ":" + stats[i].operator_name + "\n";
  }
  if (names_out != nullptr && names_len > 0) {
    std::strncpy(names_out, names.c_str(), names_len - 1);
    names_out[names_len - 1] = 0;
  }
  return MaceStatus::MACE_SUCCESS;
}

// ---- model files -------------------------------------------------------------------------

struct mbh_model {
  std::shared_ptr<MaceEngine> engine;
  std::string last_error;
};

int mbh_netdef_describe(const void *graph, size_t graph_len, char *json_out, size_t capacity, size_t *needed) {
  proto::NetDef net_def;
  MaceStatus st = ParseNetDef(graph, graph_len, &net_def);
  const std::string text = st == MaceStatus::MACE_SUCCESS ? DescribeNetDef(net_def) : st.information();
  if (needed != nullptr) *needed = text.size() + 1;
  if (json_out != nullptr && capacity > 0) {
    const size_t n = std::min(capacity - 1, text.size());
    std::memcpy(json_out, text.data(), n);
    json_out[n] = 0;
  }
  return static_cast<int>(st.code());
}

int mbh_half_to_float(const uint16_t *in, float *out, size_t count) {
  if ((in == nullptr || out == nullptr) && count != 0) return MaceStatus::MACE_INVALID_ARGS;
  for (size_t i = 0; i < count; ++i) out[i] = HalfToFloat(in[i]);
  return MaceStatus::MACE_SUCCESS;
}

int mbh_model_create(int device, const void *graph, size_t graph_len, const void *weights, size_t weights_len,
                     int fuse, int plan_memory, int cuda_graph, mbh_model **model, char *error, size_t error_len) {
  if (model == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  *model = nullptr;
  MaceEngineConfig config;
  config.SetRuntimeType(RuntimeType::RT_CUDA);
  MaceStatus cfg = config.SetCudaDevice(device);
  if (cfg != MaceStatus::MACE_SUCCESS) return static_cast<int>(cfg.code());
  config.SetCudaNetOptimizations(fuse != 0, plan_memory != 0, cuda_graph != 0);
  auto m = std::make_unique<mbh_model>();
  MaceStatus st;
  try {  // no exception may cross the C boundary
    st = CreateMaceEngineFromProto(static_cast<const unsigned char *>(graph), graph_len,
                                   static_cast<const unsigned char *>(weights), weights_len, {}, {}, config, &m->engine);
  } catch (const std::exception &ex) {
    st = MaceStatus(MaceStatus::MACE_OUT_OF_RESOURCES, std::string("exception while loading the model: ") + ex.what());
  }
  if (st != MaceStatus::MACE_SUCCESS) {
    if (error != nullptr && error_len > 0) {
      std::strncpy(error, st.information().c_str(), error_len - 1);
      error[error_len - 1] = 0;
    }
    return static_cast<int>(st.code());
  }
  *model = m.release();
  return MaceStatus::MACE_SUCCESS;
}

int mbh_model_destroy(mbh_model *model) {
  if (model == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  delete model;
  return MaceStatus::MACE_SUCCESS;
}

const char *mbh_model_last_error(const mbh_model *model) { return model ? model->last_error.c_str() : "null model"; }

void *mbh_model_context(mbh_model *model) { return model ? model->engine->runtime()->ctx() : nullptr; }

int mbh_model_captured(mbh_model *model) { return model != nullptr && model->engine->net()->captured() ? 1 : 0; }

int mbh_model_run(mbh_model *model, int n_inputs, const mbh_io_tensor *inputs, int n_outputs, mbh_io_tensor *outputs) {
  if (model == nullptr || n_inputs < 0 || n_outputs < 0 || (n_inputs > 0 && inputs == nullptr) ||
      (n_outputs > 0 && outputs == nullptr))
    return MaceStatus::MACE_INVALID_ARGS;
  auto no_delete = [](void *) {};
  std::map<std::string, MaceTensor> in, out;
  for (int i = 0; i < n_inputs; ++i) {
    const mbh_io_tensor &t = inputs[i];
    if (t.name == nullptr || t.rank < 0 || t.rank > 8) return MaceStatus::MACE_INVALID_ARGS;
    in[t.name] = MaceTensor(std::vector<int64_t>(t.shape, t.shape + t.rank), std::shared_ptr<void>(t.data, no_delete),
                            static_cast<DataFormat>(t.data_format), static_cast<IDataType>(t.data_type));
  }
  for (int i = 0; i < n_outputs; ++i) {
    const mbh_io_tensor &t = outputs[i];
    if (t.name == nullptr || t.rank < 0 || t.rank > 8) return MaceStatus::MACE_INVALID_ARGS;
    out[t.name] = MaceTensor(std::vector<int64_t>(t.shape, t.shape + t.rank), std::shared_ptr<void>(t.data, no_delete),
                             static_cast<DataFormat>(t.data_format), static_cast<IDataType>(t.data_type));
  }
  MaceStatus st;
  try {
    st = model->engine->Run(in, &out);
  } catch (const std::exception &ex) {
    st = MaceStatus(MaceStatus::MACE_OUT_OF_RESOURCES, std::string("exception while running the model: ") + ex.what());
  }
  if (st != MaceStatus::MACE_SUCCESS) {
    model->last_error = st.information();
    return static_cast<int>(st.code());
  }
  for (int i = 0; i < n_outputs; ++i) {
    const std::vector<int64_t> &shape = out[outputs[i].name].shape();
    if (shape.size() > 8) return MaceStatus::MACE_INVALID_ARGS;
    outputs[i].rank = static_cast<int>(shape.size());
    for (size_t k = 0; k < shape.size(); ++k) outputs[i].shape[k] = shape[k];
  }
  return MaceStatus::MACE_SUCCESS;
}

// ---- several GPUs ------------------------------------------------------------------------

struct mbh_multi {
  std::unique_ptr<MultiGpuRunner> runner;
  std::string last_error;
};

int mbh_shard_bounds(int64_t total, int parts, int index, int64_t *begin, int64_t *end) {
  if (begin == nullptr || end == nullptr || parts < 1 || index < 0 || index >= parts || total < 0)
    return MaceStatus::MACE_INVALID_ARGS;
  ShardBounds(total, parts, index, begin, end);
  return MaceStatus::MACE_SUCCESS;
}

int mbh_multi_create(int n_shards, const int *devices, const void *graph, size_t graph_len, const void *weights,
                     size_t weights_len, int fuse, int plan_memory, int cuda_graph, mbh_multi **runner, char *error,
                     size_t error_len) {
  if (runner == nullptr || n_shards < 1 || devices == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  *runner = nullptr;
  MaceEngineConfig config(RuntimeType::RT_CUDA);
  config.SetCudaNetOptimizations(fuse != 0, plan_memory != 0, cuda_graph != 0);
  auto m = std::make_unique<mbh_multi>();
  MaceStatus st;
  try {
    st = MultiGpuRunner::Create(std::vector<int>(devices, devices + n_shards),
                                static_cast<const unsigned char *>(graph), graph_len,
                                static_cast<const unsigned char *>(weights), weights_len, config, &m->runner);
  } catch (const std::exception &ex) {
    st = MaceStatus(MaceStatus::MACE_OUT_OF_RESOURCES, std::string("exception while loading the model: ") + ex.what());
  }
  if (st != MaceStatus::MACE_SUCCESS) {
    if (error != nullptr && error_len > 0) {
      std::strncpy(error, st.information().c_str(), error_len - 1);
      error[error_len - 1] = 0;
    }
    return static_cast<int>(st.code());
  }
  *runner = m.release();
  return MaceStatus::MACE_SUCCESS;
}

int mbh_multi_destroy(mbh_multi *runner) {
  if (runner == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  delete runner;
  return MaceStatus::MACE_SUCCESS;
}

const char *mbh_multi_last_error(const mbh_multi *runner) { return runner ? runner->last_error.c_str() : "null runner"; }

int mbh_multi_shards(const mbh_multi *runner) { return runner ? runner->runner->shards() : 0; }

int mbh_multi_run(mbh_multi *runner, int n_inputs, const mbh_io_tensor *inputs, int n_outputs,
                  mbh_io_tensor *outputs) {
  if (runner == nullptr || n_inputs < 1 || n_outputs < 1 || inputs == nullptr || outputs == nullptr)
    return MaceStatus::MACE_INVALID_ARGS;
  auto no_delete = [](void *) {};
  std::map<std::string, MaceTensor> in, out;
  for (int i = 0; i < n_inputs; ++i) {
    const mbh_io_tensor &t = inputs[i];
    if (t.name == nullptr || t.rank < 1 || t.rank > 8) return MaceStatus::MACE_INVALID_ARGS;
    in[t.name] = MaceTensor(std::vector<int64_t>(t.shape, t.shape + t.rank), std::shared_ptr<void>(t.data, no_delete),
                            static_cast<DataFormat>(t.data_format), static_cast<IDataType>(t.data_type));
  }
  for (int i = 0; i < n_outputs; ++i) {
    const mbh_io_tensor &t = outputs[i];
    if (t.name == nullptr || t.rank < 1 || t.rank > 8) return MaceStatus::MACE_INVALID_ARGS;
    out[t.name] = MaceTensor(std::vector<int64_t>(t.shape, t.shape + t.rank), std::shared_ptr<void>(t.data, no_delete),
                             static_cast<DataFormat>(t.data_format), static_cast<IDataType>(t.data_type));
  }
  MaceStatus st;
  try {
    st = runner->runner->Run(in, &out);
  } catch (const std::exception &ex) {
    st = MaceStatus(MaceStatus::MACE_OUT_OF_RESOURCES, std::string("exception while running the model: ") + ex.what());
  }
  if (st != MaceStatus::MACE_SUCCESS) {
    runner->last_error = st.information();
    return static_cast<int>(st.code());
  }
  for (int i = 0; i < n_outputs; ++i) {
    const std::vector<int64_t> &shape = out[outputs[i].name].shape();
    if (shape.size() > 8) return MaceStatus::MACE_INVALID_ARGS;
    outputs[i].rank = static_cast<int>(shape.size());
    for (size_t k = 0; k < shape.size(); ++k) outputs[i].shape[k] = shape[k];
  }
  return MaceStatus::MACE_SUCCESS;
}

// ---- logging -----------------------------------------------------------------------------

int mbh_set_log_sink(mbh_log_sink sink) {
  SetLogSink(sink);
  return MaceStatus::MACE_SUCCESS;
}

int mbh_set_vlog_level(int level) {
  SetVLogLevelForTest(level);
  return MaceStatus::MACE_SUCCESS;
}

int mbh_vlog_is_on(int level) { return ShouldGenerateVLogMessage(level) ? 1 : 0; }

int mbh_log(int severity, const char *message) {
  if (message == nullptr || severity < INFO || severity > ERROR) return MaceStatus::MACE_INVALID_ARGS;
  Logger(__FILE__, __LINE__, static_cast<LogLevel>(severity)) << message;
  return MaceStatus::MACE_SUCCESS;
}

int mbh_model_run_metadata(mbh_model *model, char *json_out, size_t capacity, size_t *needed) {
  if (model == nullptr) return MaceStatus::MACE_INVALID_ARGS;
  RunMetadata md;
  MaceStatus st = model->engine->net()->Run(&md);
  if (st == MaceStatus::MACE_SUCCESS) st = model->engine->runtime()->Status(mb_stream_sync(model->engine->runtime()->ctx()));
  if (st != MaceStatus::MACE_SUCCESS) {
    model->last_error = st.information();
    return static_cast<int>(st.code());
  }
  std::ostringstream ss;
  auto list = [&ss](const auto &v) {
    ss << "[";
    for (size_t i = 0; i < v.size(); ++i) ss << (i ? "," : "") << v[i];
    ss << "]";
  };
  ss << "[";
  for (size_t i = 0; i < md.op_stats.size(); ++i) {
    const OperatorStats &o = md.op_stats[i];
    ss << (i ? "," : "") << "{\"name\":\"" << o.operator_name << "\",\"type\":\"" << o.type
       << "\",\"device_ms\":" << o.device_ms << ",\"start_micros\":" << o.stats.start_micros
       << ",\"end_micros\":" << o.stats.end_micros << ",\"output_shape\":[";
    for (size_t k = 0; k < o.output_shape.size(); ++k) {
      ss << (k ? "," : "");
      list(o.output_shape[k]);
    }
    ss << "],\"strides\":";
    list(o.args.strides);
    ss << ",\"padding_type\":" << o.args.padding_type << ",\"paddings\":";
    list(o.args.paddings);
    ss << ",\"dilations\":";
    list(o.args.dilations);
    ss << ",\"kernels\":";
    list(o.args.kernels);
    ss << "}";
  }
  ss << "]";
  const std::string text = ss.str();
  if (needed != nullptr) *needed = text.size() + 1;
  if (json_out != nullptr && capacity > 0) {
    const size_t n = std::min(capacity - 1, text.size());
    std::memcpy(json_out, text.data(), n);
    json_out[n] = 0;
  }
  return MaceStatus::MACE_SUCCESS;
}

}  // extern "C"
