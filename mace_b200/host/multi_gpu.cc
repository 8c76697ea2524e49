#include "multi_gpu.h"

#include <algorithm>

#include "logging.h"

namespace mace {

void ShardBounds(int64_t total, int parts, int index, int64_t *begin, int64_t *end) {
  if (parts < 1 || index < 0 || index >= parts || total <= 0) {
    *begin = *end = 0;
    return;
  }
  const int64_t base = total / parts, extra = total % parts;
  *begin = index * base + std::min<int64_t>(index, extra);
  *end = *begin + base + (index < extra ? 1 : 0);
}

namespace {

size_t ElementBytes(IDataType dt) {
  switch (dt) {
    case IDT_FLOAT: return 4;
    case IDT_UINT8: return 1;
    case IDT_HALF: return 2;
    case IDT_INT32: return 4;
    default: return 0;
  }
}

// Rows [begin, end) of a host tensor whose first dimension is the batch, as a tensor of its own
// that points into the same buffer.
MaceTensor SliceRows(const MaceTensor &whole, int64_t begin, int64_t end) {
  std::vector<int64_t> shape = whole.shape();
  int64_t row_elems = 1;
  for (size_t i = 1; i < shape.size(); ++i) row_elems *= shape[i];
  shape[0] = end - begin;
  char *base = static_cast<char *>(whole.data<void>().get());
  std::shared_ptr<void> view(whole.data<void>(),
                             base + static_cast<size_t>(begin * row_elems) * ElementBytes(whole.data_type()));
  return MaceTensor(shape, view, whole.data_format(), whole.data_type());
}

}  // namespace

MaceStatus MultiGpuRunner::Create(const std::vector<int> &devices, const unsigned char *model_graph_proto,
                                  size_t model_graph_proto_size, const unsigned char *model_weights_data,
                                  size_t model_weights_data_size, const MaceEngineConfig &config,
                                  std::unique_ptr<MultiGpuRunner> *runner) {
  if (runner == nullptr || devices.empty()) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "no devices");
  std::unique_ptr<MultiGpuRunner> r(new MultiGpuRunner());
  r->graph_ = model_graph_proto;
  r->graph_len_ = model_graph_proto_size;
  r->weights_ = model_weights_data;
  r->weights_len_ = model_weights_data_size;
  r->config_ = config;
  r->job_ = Job::kInit;
  r->pending_ = static_cast<int>(devices.size());
  r->generation_ = 1;
  for (size_t i = 0; i < devices.size(); ++i) {
    auto w = std::make_unique<Worker>();
    w->index = static_cast<int>(i);
    w->device = devices[i];
    r->workers_.push_back(std::move(w));
  }
  for (auto &w : r->workers_) w->thread = std::thread(&MultiGpuRunner::Loop, r.get(), w.get());
  {
    std::unique_lock<std::mutex> lock(r->mutex_);
    r->done_.wait(lock, [&] { return r->pending_ == 0; });
  }
  for (auto &w : r->workers_)
    if (w->status != MaceStatus::MACE_SUCCESS)
      return MaceStatus(w->status.code(), "shard " + std::to_string(w->index) + " (device " +
                                              std::to_string(w->device) + "): " + w->status.information());
  VLOG(1) << "MultiGpuRunner: " << devices.size() << " shards ready";
  *runner = std::move(r);
  return MaceStatus::MACE_SUCCESS;
}

MultiGpuRunner::~MultiGpuRunner() {
  {
    std::lock_guard<std::mutex> lock(mutex_);
    stop_ = true;
  }
  wake_.notify_all();
  for (auto &w : workers_)
    if (w->thread.joinable()) w->thread.join();
}

void MultiGpuRunner::Loop(Worker *w) {
  uint64_t seen = 0;
  while (true) {
    Job job;
    {
      std::unique_lock<std::mutex> lock(mutex_);
      wake_.wait(lock, [&] { return stop_ || generation_ != seen; });
      if (stop_) break;
      seen = generation_;
      job = job_;
    }
    MaceStatus st;
    if (job == Job::kInit) {
      MaceEngineConfig cfg = config_;
      st = cfg.SetCudaDevice(w->device);
      if (st == MaceStatus::MACE_SUCCESS)
        st = CreateMaceEngineFromProto(graph_, graph_len_, weights_, weights_len_, {}, {}, cfg, &w->engine);
    } else {
      st = RunShard(w);
    }
    {
      std::lock_guard<std::mutex> lock(mutex_);
      w->status = st;
      if (--pending_ == 0) done_.notify_all();
    }
  }
  w->engine.reset();  // the engine's device memory goes away on the thread that used it
}

MaceStatus MultiGpuRunner::RunShard(Worker *w) {
  const int parts = static_cast<int>(workers_.size());
  std::map<std::string, MaceTensor> in;
  int64_t begin = 0, end = 0;
  for (const auto &kv : *inputs_) {
    ShardBounds(kv.second.shape()[0], parts, w->index, &begin, &end);
    if (begin == end) return MaceStatus::MACE_SUCCESS;  // fewer images than shards: nothing to do here
    in[kv.first] = SliceRows(kv.second, begin, end);
  }
  // This shard's rows of every output: the engine reports how many columns a row has only after
  // the run, so the view starts at the row offset implied by the caller's declared shape.
  w->outputs.clear();
  for (const auto &kv : *outputs_) w->outputs[kv.first] = SliceRows(kv.second, begin, end);
  return w->engine->Run(in, &w->outputs);
}

MaceStatus MultiGpuRunner::Run(const std::map<std::string, MaceTensor> &inputs,
                               std::map<std::string, MaceTensor> *outputs) {
  if (outputs == nullptr || inputs.empty()) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "no inputs or outputs");
  int64_t batch = -1;
  for (const auto &kv : inputs) {
    if (kv.second.shape().empty() || kv.second.data<void>() == nullptr || ElementBytes(kv.second.data_type()) == 0)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "input " + kv.first + ": needs a batch dimension and data");
    if (batch >= 0 && kv.second.shape()[0] != batch)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "inputs disagree on the batch dimension");
    batch = kv.second.shape()[0];
  }
  for (const auto &kv : *outputs) {
    if (kv.second.shape().empty() || kv.second.data<void>() == nullptr || ElementBytes(kv.second.data_type()) == 0)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "output " + kv.first + ": needs a batch dimension and a buffer");
    if (kv.second.shape()[0] < batch)
      return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "output " + kv.first + ": the buffer holds fewer rows than the batch");
  }
  {
    std::lock_guard<std::mutex> lock(mutex_);
    job_ = Job::kRun;
    inputs_ = &inputs;
    outputs_ = outputs;
    pending_ = static_cast<int>(workers_.size());
    ++generation_;
  }
  wake_.notify_all();
  {
    std::unique_lock<std::mutex> lock(mutex_);
    done_.wait(lock, [&] { return pending_ == 0; });
  }
  for (auto &w : workers_)
    if (w->status != MaceStatus::MACE_SUCCESS)
      return MaceStatus(w->status.code(), "shard " + std::to_string(w->index) + " (device " +
                                              std::to_string(w->device) + "): " + w->status.information());
  // the shape of the whole: the batch, then what a shard reported for the rest
  for (auto &kv : *outputs) {
    for (auto &w : workers_) {
      auto it = w->outputs.find(kv.first);
      if (it == w->outputs.end() || it->second.shape().empty()) continue;
      std::vector<int64_t> shape = it->second.shape();
      shape[0] = batch;
      kv.second = MaceTensor(shape, kv.second.data<void>(), kv.second.data_format(), kv.second.data_type());
      break;
    }
  }
  return MaceStatus::MACE_SUCCESS;
}

}  // namespace mace
