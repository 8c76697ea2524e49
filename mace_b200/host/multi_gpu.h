// Data-parallel inference over the GPUs of one box.  The reference has no multi-device code: a
// SerialNet runs one net on one device (mace/core/net/serial_net.cc:103-124); what it does
// support is several engines running in parallel host threads
// (test/ccunit/mace/libmace/mace_api_mt_test.cc:100-110).  This runner uses exactly that: one
// MaceEngine per shard (normally one per GPU), each with a full replica of the weights, its own
// stream and CUDA graph, driven by its own host thread.  A run splits every input along its
// first (batch) dimension into contiguous shards, each worker uploads its shard, runs its
// engine and copies its output rows device-to-host straight into its slice of the caller's
// output buffer.  No collective, no peer access: the operators are independent across images.
#ifndef MACE_B200_HOST_MULTI_GPU_H_
#define MACE_B200_HOST_MULTI_GPU_H_

#include <condition_variable>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "mace_engine.h"

namespace mace {

// Shard `index` of `parts` over `total` items: contiguous runs in order, the first
// (total % parts) shards one item longer.  Shards past the end are empty.
void ShardBounds(int64_t total, int parts, int index, int64_t *begin, int64_t *end);

class MultiGpuRunner {
 public:
  // devices[i] is the CUDA ordinal shard i runs on (an ordinal may repeat: two shards then share a
  // GPU through two engines).  The engines are created in parallel, each in its worker thread.
  static MaceStatus Create(const std::vector<int> &devices, const unsigned char *model_graph_proto,
                           size_t model_graph_proto_size, const unsigned char *model_weights_data,
                           size_t model_weights_data_size, const MaceEngineConfig &config,
                           std::unique_ptr<MultiGpuRunner> *runner);
  ~MultiGpuRunner();
  MultiGpuRunner(const MultiGpuRunner &) = delete;
  MultiGpuRunner &operator=(const MultiGpuRunner &) = delete;

  // The signature of MaceEngine::Run.  Every input's and output's first dimension is the batch;
  // all inputs must agree on it.  An output buffer must hold the rows of all shards; after the
  // run its shape() is [batch, ...].  Returns the first failing shard's status.
  MaceStatus Run(const std::map<std::string, MaceTensor> &inputs, std::map<std::string, MaceTensor> *outputs);

  int shards() const { return static_cast<int>(workers_.size()); }
  MaceEngine *engine(int shard) { return workers_[static_cast<size_t>(shard)]->engine.get(); }

 private:
  struct Worker {
    int index = 0;
    int device = 0;
    std::shared_ptr<MaceEngine> engine;
    std::thread thread;
    MaceStatus status;
    std::map<std::string, MaceTensor> outputs;  // this shard's view of the caller's buffers
  };
  MultiGpuRunner() = default;
  void Loop(Worker *w);
  MaceStatus RunShard(Worker *w);

  std::vector<std::unique_ptr<Worker>> workers_;
  std::mutex mutex_;
  std::condition_variable wake_, done_;
  uint64_t generation_ = 0;  // bumped per job; workers run once per value
  int pending_ = 0;
  bool stop_ = false;
  // the job (valid while pending_ > 0)
  enum class Job { kInit, kRun } job_ = Job::kInit;
  const std::map<std::string, MaceTensor> *inputs_ = nullptr;
  std::map<std::string, MaceTensor> *outputs_ = nullptr;
  // Init arguments
  const unsigned char *graph_ = nullptr, *weights_ = nullptr;
  size_t graph_len_ = 0, weights_len_ = 0;
  MaceEngineConfig config_;
};

}  // namespace mace

#endif  // MACE_B200_HOST_MULTI_GPU_H_
