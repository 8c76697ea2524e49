// Host-layer checks that need neither a GPU nor the device library: compiled and run by
// tests/test_host_cpu.py.  Exit code 0 = all checks passed; a failing check prints its line.
#include <cstdio>
#include <string>
#include <vector>

#include "../mace_b200/host/core.h"
#include "../mace_b200/host/delegators.h"
#include "../mace_b200/host/logging.h"
#include "../mace_b200/host/mace_engine.h"

using namespace mace;  // NOLINT

static int failures = 0;
#define EXPECT(cond)                                              \
  do {                                                            \
    if (!(cond)) {                                                \
      std::printf("line %d: %s\n", __LINE__, #cond);              \
      ++failures;                                                 \
    }                                                             \
  } while (0)

static std::vector<std::string> lines;
static void Sink(int, const char *line) { lines.push_back(line); }

namespace {
struct DummyGemm : public ops::delegator::Gemm {
  explicit DummyGemm(const ops::delegator::GemmParam &p) : Gemm(p) {}
  MaceStatus Compute(const OpContext *, const Tensor *, const Tensor *, const index_t, const index_t, const index_t,
                     const index_t, const ops::MatrixMajor, const ops::MatrixMajor, const ops::MatrixMajor, const bool, const bool,
                     Tensor *) override {
    return MaceStatus::MACE_SUCCESS;
  }
  MaceStatus Compute(const OpContext *, const Tensor *, const Tensor *, const index_t, const index_t, const index_t,
                     const index_t, const index_t, const bool, const bool, const bool, const bool, const bool,
                     Tensor *) override {
    return MaceStatus::MACE_SUCCESS;
  }
};
}  // namespace

int main() {
  // ---- the delegator registry: exact key, then the "general" tag, then an EMPTY creator (the
  // operator reports MACE_UNSUPPORTED; nothing aborts)
  Workspace ws;
  OpDelegatorRegistry *reg = ws.GetDelegatorRegistry();
  MACE_REGISTER_DELEGATOR(reg, DummyGemm, ops::delegator::GemmParam,
                          MACE_DELEGATOR_KEY(Gemm, RuntimeType::RT_CUDA, uint8_t, ImplType::CUDA));
  auto ok = ops::delegator::Gemm::Create(&ws, MACE_DELEGATOR_KEY(Gemm, RuntimeType::RT_CUDA, uint8_t, ImplType::CUDA),
                                         ops::delegator::GemmParam());
  EXPECT(ok != nullptr);
  auto tagged = ops::delegator::Gemm::Create(
      &ws, MACE_DELEGATOR_KEY_EX(Gemm, RuntimeType::RT_CUDA, uint8_t, ImplType::CUDA, K1x1), ops::delegator::GemmParam());
  EXPECT(tagged != nullptr);  // falls back to the untagged ("general") registration
  auto missing = ops::delegator::Gemm::Create(&ws, MACE_DELEGATOR_KEY(Gemm, RuntimeType::RT_CUDA, float, ImplType::CUDA),
                                              ops::delegator::GemmParam());
  EXPECT(missing == nullptr);
  EXPECT(reg->last_missing().find("Gemm") != std::string::npos);
  auto status_of = [&]() -> MaceStatus {
    MACE_RETURN_IF_NO_DELEGATOR(missing, &ws);
    return MaceStatus::MACE_SUCCESS;
  };
  const MaceStatus st = status_of();
  EXPECT(st.code() == MaceStatus::MACE_UNSUPPORTED);
  EXPECT(st.information().find("no delegator registered for") == 0);

  // ---- ConvType keeps the reference's numbering (mace/ops/delegator/conv_2d.h:28-41)
  EXPECT(ops::K1x1 == 0 && ops::K3x3S1 == 5 && ops::K3x3S2 == 6 && ops::K3x3Winograd == 7 && ops::K7x7S3 == 11);

  // ---- MaceEngineConfig: the reference's setters compile and an engine for another runtime fails
  MaceEngineConfig config(RuntimeType::RT_CUDA);
  config.SetRuntimeType(RuntimeType::RT_CUDA, "default_graph");
  EXPECT(config.SetCPUThreadPolicy(4, AFFINITY_BIG_ONLY) == MaceStatus::MACE_SUCCESS);
  EXPECT(config.SetGPUHints(PERF_HIGH, PRIORITY_LOW) == MaceStatus::MACE_SUCCESS);
  EXPECT(config.SetCudaDevice(-1).code() == MaceStatus::MACE_INVALID_ARGS);
  EXPECT(config.SetCudaDevice(3) == MaceStatus::MACE_SUCCESS && config.device() == 3);
  config.SetCudaNetOptimizations(true, false, true);
  EXPECT(config.fuse() && !config.plan_memory() && config.cuda_graph());
  RunMetadata md;
  md.op_stats.push_back(OperatorStats());
  EXPECT(md.op_stats[0].stats.start_micros == 0 && md.op_stats[0].args.padding_type == -1);

  // ---- logging: sink, levels, VLOG gating, latency logger
  SetLogSink(Sink);
  LOG(WARNING) << "w " << 7;
  EXPECT(lines.size() == 1 && lines[0].find("W host_unit.cc:") == 0 && lines[0].find("] w 7") != std::string::npos);
  VLOG(1) << "hidden";
  EXPECT(lines.size() == 1);  // MACE_CPP_MIN_VLOG_LEVEL is 0 unless the environment says otherwise
  SetVLogLevelForTest(2);
  VLOG(2) << "shown";
  VLOG(3) << "hidden";
  EXPECT(lines.size() == 2 && lines[1].find("I host_unit.cc:") == 0);
  {
    MACE_LATENCY_LOGGER(1, "Running net");
  }
  EXPECT(lines.size() == 4 && lines[2].find("Running net started") != std::string::npos &&
         lines[3].find("Running net latency: ") != std::string::npos);
  SetVLogLevelForTest(-1);
  VLOG(0) << "hidden";
  EXPECT(lines.size() == 4);
  std::printf("%d failures\n", failures);
  return failures == 0 ? 0 : 1;
}
