// Host-side core types of the CUDA runtime, API-compatible with the parts of
// MACE's core that the hot-path operators touch: MaceStatus, RuntimeType,
// DataType, Tensor, Runtime, OpContext, OpDelegator, the delegator registry
// and its macros.  Written from scratch against the interfaces of
//   include/mace/public/mace.h:48-58, :244-291 (RuntimeType, MaceStatus)
//   mace/core/tensor.h:103-264                 (Tensor)
//   mace/core/runtime/runtime.h:42-104         (Runtime)
//   mace/core/ops/op_delegator.h:25-54         (OpDelegator, ImplType)
//   mace/core/registry/op_delegator_registry.h:32-125 (registry + macros)
// so that delegators and operators written for MACE compile against it with
// the same names and argument meanings.  Tensors of this runtime live in
// device memory; data<T>() is not offered on purpose (no host mapping on the
// hot path), memory<T>() returns the device pointer as in MACE's device
// runtimes (mace/core/memory/buffer.h:41-59).
#ifndef MACE_B200_HOST_CORE_H_
#define MACE_B200_HOST_CORE_H_

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/mace_b200.h"

namespace mace {

typedef int64_t index_t;

enum RuntimeType {
  RT_CPU = 0,
  RT_OPENCL = 2,
  RT_HEXAGON = 3,
  RT_HTA = 4,
  RT_APU = 5,
  RT_HTP = 6,
  RT_CUDA = 7,  // new: this runtime
  RT_NONE = 65534,
  RT_MAX = 65535,
};

enum DataType {  // mace/proto/mace.proto:10-23
  DT_INVALID = 0,
  DT_FLOAT = 1,
  DT_UINT8 = 2,
  DT_HALF = 3,
  DT_INT32 = 4,
};

enum class DataFormat { NONE = 0, NHWC = 1, NCHW = 2, HWOI = 100, OIHW = 101, HWIO = 102, OHWI = 103, AUTO = 1000 };

enum ImplType { REF = 0, NEON, CUDA };

inline size_t GetEnumTypeSize(DataType dt) {
  switch (dt) {
    case DT_FLOAT: return 4;
    case DT_UINT8: return 1;
    case DT_HALF: return 2;
    case DT_INT32: return 4;
    default: return 0;
  }
}

template <typename T> struct DataTypeToEnum;
template <> struct DataTypeToEnum<float> { static constexpr DataType value = DT_FLOAT; static DataType v() { return value; } };
template <> struct DataTypeToEnum<uint8_t> { static constexpr DataType value = DT_UINT8; static DataType v() { return value; } };
template <> struct DataTypeToEnum<int32_t> { static constexpr DataType value = DT_INT32; static DataType v() { return value; } };

class MaceStatus {
 public:
  enum Code {
    MACE_SUCCESS = 0,
    MACE_INVALID_ARGS = 1,
    MACE_OUT_OF_RESOURCES = 2,
    MACE_UNSUPPORTED = 3,
    MACE_RUNTIME_ERROR = 4,
  };
  MaceStatus() : code_(MACE_SUCCESS) {}
  MaceStatus(const Code code) : code_(code) {}  // NOLINT(runtime/explicit)
  MaceStatus(const Code code, const std::string &information) : code_(code), info_(information) {}
  Code code() const { return code_; }
  std::string information() const { return info_; }
  bool operator==(const MaceStatus &other) const { return code_ == other.code_; }
  bool operator!=(const MaceStatus &other) const { return code_ != other.code_; }

 private:
  Code code_;
  std::string info_;
};

#define MACE_RETURN_IF_ERROR(stmt)                          \
  do {                                                      \
    ::mace::MaceStatus _status = (stmt);                    \
    if (_status != ::mace::MaceStatus::MACE_SUCCESS) return _status; \
  } while (0)

// Precondition violations abort, as MACE_CHECK -> LOG(FATAL) does
// (include/mace/utils/logging.h:51-95).
#define MACE_CHECK(cond, ...)                                                     \
  do {                                                                            \
    if (!(cond)) {                                                                \
      std::fprintf(stderr, "%s:%d Check failed: %s\n", __FILE__, __LINE__, #cond); \
      std::abort();                                                               \
    }                                                                             \
  } while (0)
#define MACE_CHECK_NOTNULL(ptr) MACE_CHECK((ptr) != nullptr)
// An operator whose delegator key has no registration reports it instead of aborting.
#define MACE_RETURN_IF_NO_DELEGATOR(ptr, workspace)                                              \
  do {                                                                                           \
    if ((ptr) == nullptr)                                                                        \
      return ::mace::MaceStatus(::mace::MaceStatus::MACE_UNSUPPORTED,                            \
                                "no delegator registered for " +                                 \
                                    (workspace)->GetDelegatorRegistry()->last_missing());        \
  } while (0)
#define MACE_UNUSED(x) (void)(x)

// ---- Runtime ------------------------------------------------------------------

class Runtime {
 public:
  virtual ~Runtime() = default;
  virtual RuntimeType GetRuntimeType() = 0;
  virtual MaceStatus New(size_t bytes, void **ptr) = 0;
  virtual void Delete(void *ptr) = 0;
};

// The CUDA runtime: one mb_context (stream + scratch arena) per engine, the
// counterpart of CpuRuntime (mace/runtimes/cpu/cpu_runtime.cc:28-109).
class CudaRuntime : public Runtime {
 public:
  CudaRuntime() = default;
  ~CudaRuntime() override;
  MaceStatus Init(int device);
  RuntimeType GetRuntimeType() override { return RuntimeType::RT_CUDA; }
  MaceStatus New(size_t bytes, void **ptr) override;
  void Delete(void *ptr) override;
  mb_context *ctx() const { return ctx_; }
  // Wraps a C-ABI return code with the library's message.
  MaceStatus Status(int rc) const;

 private:
  mb_context *ctx_ = nullptr;
};

class OpContext {
 public:
  explicit OpContext(Runtime *runtime) : runtime_(runtime) {}
  Runtime *runtime() const { return runtime_; }

 private:
  Runtime *runtime_;
};

inline CudaRuntime *CudaRuntimeOf(const OpContext *context) {
  MACE_CHECK(context->runtime()->GetRuntimeType() == RuntimeType::RT_CUDA);
  return static_cast<CudaRuntime *>(context->runtime());
}

// ---- Tensor ---------------------------------------------------------------------

class Tensor {
 public:
  Tensor(Runtime *runtime, DataType dtype, const std::vector<index_t> &shape = {},
         bool is_weight = false, const std::string &name = "")
      : runtime_(runtime), dtype_(dtype), is_weight_(is_weight), name_(name) {
    if (!shape.empty()) Resize(shape);
  }
  ~Tensor() {
    if (buffer_ != nullptr && owns_buffer_) runtime_->Delete(buffer_);
  }
  Tensor(const Tensor &) = delete;
  Tensor &operator=(const Tensor &) = delete;

  const std::string &name() const { return name_; }
  DataType dtype() const { return dtype_; }
  const std::vector<index_t> &shape() const { return shape_; }
  index_t dim_size() const { return static_cast<index_t>(shape_.size()); }
  index_t dim(unsigned int index) const {
    MACE_CHECK(index < shape_.size());
    return shape_[index];
  }
  index_t size() const {
    index_t n = 1;
    for (index_t d : shape_) n *= d;
    return n;
  }
  index_t raw_size() const { return size() * static_cast<index_t>(GetEnumTypeSize(dtype_)); }
  bool is_weight() const { return is_weight_; }
  float scale() const { return scale_; }
  int32_t zero_point() const { return zero_point_; }
  void SetScale(float scale) { scale_ = scale; }
  void SetZeroPoint(int32_t zero_point) { zero_point_ = zero_point; }

  // Device pointers (mace/core/tensor.h: memory<T>() / mutable_memory<T>()).
  template <typename T> const T *memory() const { return static_cast<const T *>(buffer_); }
  template <typename T> T *mutable_memory() { return static_cast<T *>(buffer_); }

  // On failure (the allocator is out of memory) the tensor keeps its old shape and memory, so
  // that a caller that retries later finds a consistent tensor.
  MaceStatus Resize(const std::vector<index_t> &shape) {
    size_t need = GetEnumTypeSize(dtype_);
    for (index_t d : shape) need *= static_cast<size_t>(d);
    if (need > capacity_) {
      void *fresh = nullptr;
      MACE_RETURN_IF_ERROR(runtime_->New(need, &fresh));
      // (a tensor that outgrows a shared buffer leaves it and owns its memory again)
      if (buffer_ != nullptr && owns_buffer_) runtime_->Delete(buffer_);
      buffer_ = fresh;
      capacity_ = need;
      owns_buffer_ = true;
    }
    shape_ = shape;
    return MaceStatus::MACE_SUCCESS;
  }

  // Memory planning (the RENT_SHARE buffers of mace/core/net/allocate_opt_strategy.cc:157-178):
  // the tensor gives up its own allocation and lives in `buffer`, which the net owns and
  // shares among tensors whose lifetimes do not overlap.  The contents are not kept.
  void BindShared(void *buffer, size_t capacity) {
    if (buffer_ != nullptr && owns_buffer_) runtime_->Delete(buffer_);
    buffer_ = buffer;
    capacity_ = capacity;
    owns_buffer_ = false;
  }
  bool owns_buffer() const { return owns_buffer_; }

 private:
  Runtime *runtime_;
  DataType dtype_;
  std::vector<index_t> shape_;
  void *buffer_ = nullptr;
  size_t capacity_ = 0;
  bool owns_buffer_ = true;
  bool is_weight_;
  float scale_ = 0.f;
  int32_t zero_point_ = 0;
  std::string name_;
};

// ---- delegators -------------------------------------------------------------------

struct DelegatorParam {
  DelegatorParam() = default;
  virtual ~DelegatorParam() = default;
};

class OpDelegator {
 public:
  explicit OpDelegator(const DelegatorParam &param) { MACE_UNUSED(param); }
  virtual ~OpDelegator() = default;

  template <class DerivedType, class ParamType>
  static std::unique_ptr<OpDelegator> DefaultCreator(const DelegatorParam &param) {
    return std::make_unique<DerivedType>(static_cast<const ParamType &>(param));
  }
};

typedef std::function<std::unique_ptr<OpDelegator>(const DelegatorParam &)> DelegatorCreator;

struct DelegatorInfo {
  DelegatorInfo(const char *name, DataType dt, RuntimeType rt, ImplType impl, const char *tag_in = "general")
      : delegator_name(name), data_type(dt), runtime(rt), impl_type(impl), tag(tag_in) {}
  std::string ToString() const {
    std::stringstream ss;
    ss << delegator_name << "_" << data_type << "_" << runtime << "_" << impl_type << "_" << tag;
    return ss.str();
  }
  bool operator==(const DelegatorInfo &o) const {
    return runtime == o.runtime && impl_type == o.impl_type && data_type == o.data_type &&
           delegator_name == o.delegator_name && tag == o.tag;
  }
  std::string delegator_name;
  DataType data_type;
  RuntimeType runtime;
  ImplType impl_type;
  std::string tag;
};

// Lookup with the reference's fall-back order: exact key, then the "general"
// tag of the same implementation (mace/core/registry/op_delegator_registry.cc:64-102).
class OpDelegatorRegistry {
 public:
  MaceStatus Register(const DelegatorInfo &key, DelegatorCreator creator) {
    MACE_CHECK(registry_.count(key.ToString()) == 0);
    registry_[key.ToString()] = std::move(creator);
    return MaceStatus::MACE_SUCCESS;
  }
  DelegatorCreator GetCreator(const DelegatorInfo &key) const {
    auto it = registry_.find(key.ToString());
    if (it != registry_.end()) return it->second;
    DelegatorInfo general = key;
    general.tag = "general";
    it = registry_.find(general.ToString());
    if (it != registry_.end()) return it->second;
    // Unknown key: an empty creator.  Delegator::Create then returns null and the operator
    // reports MACE_UNSUPPORTED (the reference aborts here, op_delegator_registry.cc:64-102;
    // behind a C boundary that would take the caller's process down).
    last_missing_ = key.ToString();
    return DelegatorCreator();
  }
  const std::string &last_missing() const { return last_missing_; }

 private:
  mutable std::string last_missing_;
  std::unordered_map<std::string, DelegatorCreator> registry_;
};

class Workspace {
 public:
  OpDelegatorRegistry *GetDelegatorRegistry() { return &delegator_registry_; }
  Tensor *CreateTensor(const std::string &name, Runtime *runtime, DataType dt, bool is_weight = false) {
    tensors_[name] = std::make_unique<Tensor>(runtime, dt, std::vector<index_t>{}, is_weight, name);
    return tensors_[name].get();
  }
  Tensor *GetTensor(const std::string &name) {
    auto it = tensors_.find(name);
    return it == tensors_.end() ? nullptr : it->second.get();
  }
  bool HasTensor(const std::string &name) const { return tensors_.count(name) != 0; }

 private:
  OpDelegatorRegistry delegator_registry_;
  std::map<std::string, std::unique_ptr<Tensor>> tensors_;
};

#define MACE_DELEGATOR_KEY_EX(delegator_name, device, DT, impl, tag) \
  ::mace::DelegatorInfo(#delegator_name, ::mace::DataTypeToEnum<DT>::value, device, impl, #tag)
#define MACE_DELEGATOR_KEY(delegator_name, device, DT, impl) \
  ::mace::DelegatorInfo(#delegator_name, ::mace::DataTypeToEnum<DT>::value, device, impl)
#define MACE_REGISTER_DELEGATOR(registry, class_name, param_name, key) \
  registry->Register(key, ::mace::OpDelegator::DefaultCreator<class_name, param_name>)
#define MACE_DEFINE_DELEGATOR_CREATOR(class_name)                                         \
  static std::unique_ptr<class_name> Create(::mace::Workspace *workspace,                  \
                                            const ::mace::DelegatorInfo &key,              \
                                            const ::mace::DelegatorParam &param) {         \
    ::mace::DelegatorCreator creator = workspace->GetDelegatorRegistry()->GetCreator(key); \
    if (!creator) return nullptr;                                                          \
    std::unique_ptr<::mace::OpDelegator> delegator = creator(param);                       \
    return std::unique_ptr<class_name>(static_cast<class_name *>(delegator.release()));    \
  }

}  // namespace mace

#endif  // MACE_B200_HOST_CORE_H_
