// Reader of MACE model files: the serialized NetDef message of mace/proto/mace.proto:25-117
// (proto2 wire format), decoded by hand so that no protobuf library and no generated
// mace.pb.h are needed.  The structs below mirror the messages field by field (the field
// numbers are in netdef.cc); unknown fields are skipped the way protobuf's lite runtime
// skips them, so files written by a newer converter still load.
#ifndef MACE_B200_HOST_NETDEF_H_
#define MACE_B200_HOST_NETDEF_H_

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "ops.h"

namespace mace {
namespace proto {

struct Argument {  // mace.proto:42-49
  std::string name;
  bool has_f = false, has_i = false, has_s = false;
  float f = 0.f;
  int64_t i = 0;
  std::string s;
  std::vector<float> floats;
  std::vector<int64_t> ints;
};

struct ConstTensor {  // mace.proto:25-40
  std::vector<int64_t> dims;
  int data_type = DT_FLOAT;
  std::vector<float> float_data;
  std::vector<int32_t> int32_data;
  std::string name;
  int64_t offset = 0;
  int64_t data_size = 0;
  float scale = 0.f;
  int32_t zero_point = 0;
  float minval = 0.f;
  float maxval = 0.f;
  bool quantized = false;
  uint32_t node_id = 0;
};

struct NodeInput {  // mace.proto:52-55
  int32_t node_id = 0;
  int32_t output_port = 0;
};

struct OutputShape {  // mace.proto:57-59
  std::vector<int64_t> dims;
};

struct QuantizeActivationInfo {  // mace.proto:61-66
  float scale = 0.f;
  int32_t zero_point = 0;
  float minval = 0.f;
  float maxval = 0.f;
};

struct OperatorDef {  // mace.proto:68-88
  std::vector<std::string> input;
  std::vector<std::string> output;
  std::string name;
  std::string type;
  int32_t device_type = 0;
  std::vector<Argument> arg;
  std::vector<OutputShape> output_shape;
  std::vector<int> output_type;
  std::vector<QuantizeActivationInfo> quantize_info;
  std::vector<int32_t> mem_id;
  uint32_t node_id = 0;
  uint32_t op_id = 0;
  uint32_t padding = 0;
  std::vector<NodeInput> node_input;
  std::vector<int32_t> out_max_byte_size;
};

struct InputOutputInfo {  // mace.proto:90-101
  std::string name;
  int32_t node_id = 0;
  std::vector<int32_t> dims;
  int32_t max_byte_size = 0;
  int data_type = DT_FLOAT;
  int32_t data_format = 1;  // NHWC
  float scale = 0.f;
  int32_t zero_point = 0;
  std::string alias;
};

struct NetDef {  // mace.proto:103-117
  std::vector<OperatorDef> op;
  std::vector<Argument> arg;
  std::vector<ConstTensor> tensors;
  int data_type = DT_FLOAT;
  std::string name;
  int32_t data_offset = 0;
  int32_t data_size = 0;
  int32_t infer_order = 0;
  std::vector<InputOutputInfo> input_info;
  std::vector<InputOutputInfo> output_info;
};

}  // namespace proto

// Decodes one serialized NetDef.  MACE_INVALID_ARGS (with the byte offset in the message)
// for truncated input, over-long varints, lengths that run past the end, group wire types
// or a wire type that does not fit the field.
MaceStatus ParseNetDef(const void *data, size_t size, proto::NetDef *net_def);

// A JSON rendering of a parsed NetDef (every field, floats with 9 significant digits), for
// tests and for inspecting a model file.
std::string DescribeNetDef(const proto::NetDef &net_def);

// ProtoArgHelper::GetOptionalArg<NetDef, int> (mace/core/proto/arg_helper.cc:50-94).
int GetNetArgInt(const proto::NetDef &net_def, const std::string &name, int default_value);

// proto::OperatorDef -> the OperatorDef the operators of this library are constructed from:
// each Argument lands in the typed map its set fields name (i, f, s, ints, floats).
void ConvertOperatorDef(const proto::OperatorDef &src, OperatorDef *dst);

// IEEE binary16 -> binary32 (the half_float::half_cast the CPU runtime applies to DT_HALF
// weights, mace/core/workspace.cc:147-157).
float HalfToFloat(uint16_t h);

}  // namespace mace

#endif  // MACE_B200_HOST_NETDEF_H_
