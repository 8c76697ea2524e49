#include "netdef.h"

#include <cstdio>
#include <cstring>
#include <sstream>

namespace mace {

namespace {

// proto2 wire types
enum WireType { WT_VARINT = 0, WT_FIXED64 = 1, WT_BYTES = 2, WT_GROUP_START = 3, WT_GROUP_END = 4, WT_FIXED32 = 5 };

// A cursor over one message (or one length-delimited field).  Every read checks the bounds;
// after a failed read ok() is false and error() names the offset within the outermost buffer.
class Reader {
 public:
  Reader(const uint8_t *base, const uint8_t *begin, const uint8_t *end) : base_(base), p_(begin), end_(end) {}
  bool done() const { return p_ >= end_; }
  bool ok() const { return error_.empty(); }
  const std::string &error() const { return error_; }
  void Adopt(const Reader &sub) {
    if (!sub.ok() && error_.empty()) error_ = sub.error_;
  }

  bool Fail(const char *what) {
    if (error_.empty()) {
      std::stringstream ss;
      ss << what << " at byte " << (p_ - base_);
      error_ = ss.str();
    }
    p_ = end_;
    return false;
  }

  bool Varint(uint64_t *value) {
    uint64_t v = 0;
    for (int shift = 0; shift < 70; shift += 7) {
      if (p_ >= end_) return Fail("truncated varint");
      const uint8_t b = *p_++;
      if (shift == 63 && (b & 0xfe) != 0) return Fail("varint longer than 64 bits");
      v |= static_cast<uint64_t>(b & 0x7f) << shift;
      if ((b & 0x80) == 0) {
        *value = v;
        return true;
      }
    }
    return Fail("varint longer than 10 bytes");
  }

  bool Tag(uint32_t *field, int *wire_type) {
    uint64_t t = 0;
    if (!Varint(&t)) return false;
    if (t > 0xffffffffull || (t >> 3) == 0) return Fail("invalid field tag");
    *field = static_cast<uint32_t>(t >> 3);
    *wire_type = static_cast<int>(t & 7);
    return true;
  }

  bool Fixed32(uint32_t *value) {
    if (end_ - p_ < 4) return Fail("truncated 32-bit value");
    std::memcpy(value, p_, 4);  // little endian on the wire and on this host
    p_ += 4;
    return true;
  }

  bool Fixed64(uint64_t *value) {
    if (end_ - p_ < 8) return Fail("truncated 64-bit value");
    std::memcpy(value, p_, 8);
    p_ += 8;
    return true;
  }

  // The payload of a length-delimited field as a reader of its own.
  bool Sub(Reader *sub) {
    uint64_t len = 0;
    if (!Varint(&len)) return false;
    if (len > static_cast<uint64_t>(end_ - p_)) return Fail("length-delimited field runs past the end");
    *sub = Reader(base_, p_, p_ + len);
    p_ += len;
    return true;
  }

  bool String(std::string *s) {
    Reader sub(base_, p_, p_);
    if (!Sub(&sub)) return false;
    s->assign(reinterpret_cast<const char *>(sub.p_), static_cast<size_t>(sub.end_ - sub.p_));
    return true;
  }

  bool Skip(int wire_type) {
    uint64_t v64 = 0;
    uint32_t v32 = 0;
    Reader sub(base_, p_, p_);
    switch (wire_type) {
      case WT_VARINT: return Varint(&v64);
      case WT_FIXED64: return Fixed64(&v64);
      case WT_BYTES: return Sub(&sub);
      case WT_FIXED32: return Fixed32(&v32);
      default: return Fail("group wire types are not part of mace.proto");
    }
  }

 private:
  const uint8_t *base_;
  const uint8_t *p_;
  const uint8_t *end_;
  std::string error_;
};

// ---- scalar fields (the last occurrence wins, as in protobuf) -------------------------

template <typename T>
bool ReadVarintField(Reader *r, int wt, T *out) {
  if (wt != WT_VARINT) return r->Fail("wire type does not fit a varint field");
  uint64_t v = 0;
  if (!r->Varint(&v)) return false;
  *out = static_cast<T>(v);  // int32 / int64 / enum: two's complement truncation; bool: != 0 below
  return true;
}

bool ReadBoolField(Reader *r, int wt, bool *out) {
  uint64_t v = 0;
  if (!ReadVarintField(r, wt, &v)) return false;
  *out = v != 0;
  return true;
}

bool ReadFloatField(Reader *r, int wt, float *out) {
  if (wt != WT_FIXED32) return r->Fail("wire type does not fit a float field");
  uint32_t bits = 0;
  if (!r->Fixed32(&bits)) return false;
  std::memcpy(out, &bits, 4);
  return true;
}

bool ReadStringField(Reader *r, int wt, std::string *out) {
  if (wt != WT_BYTES) return r->Fail("wire type does not fit a string field");
  return r->String(out);
}

// ---- repeated scalar fields: packed or one element per tag, both accepted ----------------

template <typename T>
bool ReadRepeatedVarint(Reader *r, int wt, std::vector<T> *out) {
  if (wt == WT_VARINT) {
    uint64_t v = 0;
    if (!r->Varint(&v)) return false;
    out->push_back(static_cast<T>(v));
    return true;
  }
  if (wt != WT_BYTES) return r->Fail("wire type does not fit a repeated varint field");
  Reader sub(nullptr, nullptr, nullptr);
  if (!r->Sub(&sub)) return false;
  while (!sub.done()) {
    uint64_t v = 0;
    if (!sub.Varint(&v)) break;
    out->push_back(static_cast<T>(v));
  }
  r->Adopt(sub);
  return sub.ok() ? true : r->Fail("bad packed field");
}

bool ReadRepeatedFloat(Reader *r, int wt, std::vector<float> *out) {
  if (wt == WT_FIXED32) {
    float f = 0.f;
    if (!ReadFloatField(r, wt, &f)) return false;
    out->push_back(f);
    return true;
  }
  if (wt != WT_BYTES) return r->Fail("wire type does not fit a repeated float field");
  Reader sub(nullptr, nullptr, nullptr);
  if (!r->Sub(&sub)) return false;
  while (!sub.done()) {
    float f = 0.f;
    if (!ReadFloatField(&sub, WT_FIXED32, &f)) break;
    out->push_back(f);
  }
  r->Adopt(sub);
  return sub.ok() ? true : r->Fail("bad packed field");
}

// A message-typed field: parse(sub-reader, message).
template <typename M, typename F>
bool ReadMessageField(Reader *r, int wt, M *msg, F parse) {
  if (wt != WT_BYTES) return r->Fail("wire type does not fit a message field");
  Reader sub(nullptr, nullptr, nullptr);
  if (!r->Sub(&sub)) return false;
  parse(&sub, msg);
  r->Adopt(sub);
  return sub.ok() ? true : r->Fail("bad embedded message");
}

// ---- the messages (field numbers from mace/proto/mace.proto) ----------------------------

void ParseArgument(Reader *r, proto::Argument *m) {
  uint32_t field = 0;
  int wt = 0;
  while (!r->done() && r->Tag(&field, &wt)) {
    switch (field) {
      case 1: ReadStringField(r, wt, &m->name); break;
      case 2: m->has_f = ReadFloatField(r, wt, &m->f) || m->has_f; break;
      case 3: m->has_i = ReadVarintField(r, wt, &m->i) || m->has_i; break;
      case 4: m->has_s = ReadStringField(r, wt, &m->s) || m->has_s; break;
      case 5: ReadRepeatedFloat(r, wt, &m->floats); break;
      case 6: ReadRepeatedVarint(r, wt, &m->ints); break;
      default: r->Skip(wt);
    }
  }
}

void ParseConstTensor(Reader *r, proto::ConstTensor *m) {
  uint32_t field = 0;
  int wt = 0;
  while (!r->done() && r->Tag(&field, &wt)) {
    switch (field) {
      case 1: ReadRepeatedVarint(r, wt, &m->dims); break;
      case 2: ReadVarintField(r, wt, &m->data_type); break;
      case 3: ReadRepeatedFloat(r, wt, &m->float_data); break;
      case 4: ReadRepeatedVarint(r, wt, &m->int32_data); break;
      case 5: ReadStringField(r, wt, &m->name); break;
      case 6: ReadVarintField(r, wt, &m->offset); break;
      case 7: ReadVarintField(r, wt, &m->data_size); break;
      case 8: ReadFloatField(r, wt, &m->scale); break;
      case 9: ReadVarintField(r, wt, &m->zero_point); break;
      case 10: ReadFloatField(r, wt, &m->minval); break;
      case 11: ReadFloatField(r, wt, &m->maxval); break;
      case 12: ReadBoolField(r, wt, &m->quantized); break;
      case 100: ReadVarintField(r, wt, &m->node_id); break;
      default: r->Skip(wt);
    }
  }
}

void ParseNodeInput(Reader *r, proto::NodeInput *m) {
  uint32_t field = 0;
  int wt = 0;
  while (!r->done() && r->Tag(&field, &wt)) {
    switch (field) {
      case 1: ReadVarintField(r, wt, &m->node_id); break;
      case 2: ReadVarintField(r, wt, &m->output_port); break;
      default: r->Skip(wt);
    }
  }
}

void ParseOutputShape(Reader *r, proto::OutputShape *m) {
  uint32_t field = 0;
  int wt = 0;
  while (!r->done() && r->Tag(&field, &wt)) {
    if (field == 1) ReadRepeatedVarint(r, wt, &m->dims);
    else r->Skip(wt);
  }
}

void ParseQuantizeInfo(Reader *r, proto::QuantizeActivationInfo *m) {
  uint32_t field = 0;
  int wt = 0;
  while (!r->done() && r->Tag(&field, &wt)) {
    switch (field) {
      case 1: ReadFloatField(r, wt, &m->scale); break;
      case 2: ReadVarintField(r, wt, &m->zero_point); break;
      case 3: ReadFloatField(r, wt, &m->minval); break;
      case 4: ReadFloatField(r, wt, &m->maxval); break;
      default: r->Skip(wt);
    }
  }
}

void ParseOperatorDef(Reader *r, proto::OperatorDef *m) {
  uint32_t field = 0;
  int wt = 0;
  std::string s;
  while (!r->done() && r->Tag(&field, &wt)) {
    switch (field) {
      case 1:
        if (ReadStringField(r, wt, &s)) m->input.push_back(s);
        break;
      case 2:
        if (ReadStringField(r, wt, &s)) m->output.push_back(s);
        break;
      case 3: ReadStringField(r, wt, &m->name); break;
      case 4: ReadStringField(r, wt, &m->type); break;
      case 5: ReadVarintField(r, wt, &m->device_type); break;
      case 6:
        m->arg.emplace_back();
        ReadMessageField(r, wt, &m->arg.back(), ParseArgument);
        break;
      case 7:
        m->output_shape.emplace_back();
        ReadMessageField(r, wt, &m->output_shape.back(), ParseOutputShape);
        break;
      case 8: ReadRepeatedVarint(r, wt, &m->output_type); break;
      case 9:
        m->quantize_info.emplace_back();
        ReadMessageField(r, wt, &m->quantize_info.back(), ParseQuantizeInfo);
        break;
      case 10: ReadRepeatedVarint(r, wt, &m->mem_id); break;
      case 100: ReadVarintField(r, wt, &m->node_id); break;
      case 101: ReadVarintField(r, wt, &m->op_id); break;
      case 102: ReadVarintField(r, wt, &m->padding); break;
      case 103:
        m->node_input.emplace_back();
        ReadMessageField(r, wt, &m->node_input.back(), ParseNodeInput);
        break;
      case 104: ReadRepeatedVarint(r, wt, &m->out_max_byte_size); break;
      default: r->Skip(wt);
    }
  }
}

void ParseInputOutputInfo(Reader *r, proto::InputOutputInfo *m) {
  uint32_t field = 0;
  int wt = 0;
  while (!r->done() && r->Tag(&field, &wt)) {
    switch (field) {
      case 1: ReadStringField(r, wt, &m->name); break;
      case 2: ReadVarintField(r, wt, &m->node_id); break;
      case 3: ReadRepeatedVarint(r, wt, &m->dims); break;
      case 4: ReadVarintField(r, wt, &m->max_byte_size); break;
      case 5: ReadVarintField(r, wt, &m->data_type); break;
      case 6: ReadVarintField(r, wt, &m->data_format); break;
      case 7: ReadFloatField(r, wt, &m->scale); break;
      case 8: ReadVarintField(r, wt, &m->zero_point); break;
      case 100: ReadStringField(r, wt, &m->alias); break;
      default: r->Skip(wt);
    }
  }
}

void ParseNetDefMessage(Reader *r, proto::NetDef *m) {
  uint32_t field = 0;
  int wt = 0;
  while (!r->done() && r->Tag(&field, &wt)) {
    switch (field) {
      case 1:
        m->op.emplace_back();
        ReadMessageField(r, wt, &m->op.back(), ParseOperatorDef);
        break;
      case 2:
        m->arg.emplace_back();
        ReadMessageField(r, wt, &m->arg.back(), ParseArgument);
        break;
      case 3:
        m->tensors.emplace_back();
        ReadMessageField(r, wt, &m->tensors.back(), ParseConstTensor);
        break;
      case 4: ReadVarintField(r, wt, &m->data_type); break;
      case 5: ReadStringField(r, wt, &m->name); break;
      case 6: ReadVarintField(r, wt, &m->data_offset); break;
      case 7: ReadVarintField(r, wt, &m->data_size); break;
      case 8: ReadVarintField(r, wt, &m->infer_order); break;
      case 100:
        m->input_info.emplace_back();
        ReadMessageField(r, wt, &m->input_info.back(), ParseInputOutputInfo);
        break;
      case 101:
        m->output_info.emplace_back();
        ReadMessageField(r, wt, &m->output_info.back(), ParseInputOutputInfo);
        break;
      default: r->Skip(wt);
    }
  }
}

// ---- JSON rendering -------------------------------------------------------------------------

void JsonString(std::stringstream &ss, const std::string &s) {
  ss << '"';
  for (unsigned char c : s) {
    if (c == '"' || c == '\\') {
      ss << '\\' << c;
    } else if (c < 0x20 || c >= 0x7f) {
      char buf[8];
      std::snprintf(buf, sizeof(buf), "\\u%04x", c);
      ss << buf;
    } else {
      ss << c;
    }
  }
  ss << '"';
}

void JsonFloat(std::stringstream &ss, float f) {
  char buf[32];
  std::snprintf(buf, sizeof(buf), "%.9g", static_cast<double>(f));
  ss << buf;
}

template <typename T>
void JsonInts(std::stringstream &ss, const std::vector<T> &v) {
  ss << '[';
  for (size_t i = 0; i < v.size(); ++i) ss << (i ? "," : "") << static_cast<int64_t>(v[i]);
  ss << ']';
}

void JsonFloats(std::stringstream &ss, const std::vector<float> &v) {
  ss << '[';
  for (size_t i = 0; i < v.size(); ++i) {
    if (i) ss << ',';
    JsonFloat(ss, v[i]);
  }
  ss << ']';
}

void JsonStrings(std::stringstream &ss, const std::vector<std::string> &v) {
  ss << '[';
  for (size_t i = 0; i < v.size(); ++i) {
    if (i) ss << ',';
    JsonString(ss, v[i]);
  }
  ss << ']';
}

void JsonArgument(std::stringstream &ss, const proto::Argument &a) {
  ss << "{\"name\":";
  JsonString(ss, a.name);
  if (a.has_f) {
    ss << ",\"f\":";
    JsonFloat(ss, a.f);
  }
  if (a.has_i) ss << ",\"i\":" << a.i;
  if (a.has_s) {
    ss << ",\"s\":";
    JsonString(ss, a.s);
  }
  if (!a.floats.empty()) {
    ss << ",\"floats\":";
    JsonFloats(ss, a.floats);
  }
  if (!a.ints.empty()) {
    ss << ",\"ints\":";
    JsonInts(ss, a.ints);
  }
  ss << '}';
}

void JsonInfo(std::stringstream &ss, const proto::InputOutputInfo &m) {
  ss << "{\"name\":";
  JsonString(ss, m.name);
  ss << ",\"node_id\":" << m.node_id << ",\"dims\":";
  JsonInts(ss, m.dims);
  ss << ",\"max_byte_size\":" << m.max_byte_size << ",\"data_type\":" << m.data_type
     << ",\"data_format\":" << m.data_format << ",\"scale\":";
  JsonFloat(ss, m.scale);
  ss << ",\"zero_point\":" << m.zero_point << ",\"alias\":";
  JsonString(ss, m.alias);
  ss << '}';
}

}  // namespace

MaceStatus ParseNetDef(const void *data, size_t size, proto::NetDef *net_def) {
  if (net_def == nullptr || (data == nullptr && size != 0))
    return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "null NetDef buffer");
  *net_def = proto::NetDef();
  const uint8_t *p = static_cast<const uint8_t *>(data);
  Reader r(p, p, p + size);
  ParseNetDefMessage(&r, net_def);
  if (!r.ok()) return MaceStatus(MaceStatus::MACE_INVALID_ARGS, "malformed NetDef: " + r.error());
  return MaceStatus::MACE_SUCCESS;
}

std::string DescribeNetDef(const proto::NetDef &n) {
  std::stringstream ss;
  ss << "{\"name\":";
  JsonString(ss, n.name);
  ss << ",\"data_type\":" << n.data_type << ",\"data_offset\":" << n.data_offset << ",\"data_size\":" << n.data_size
     << ",\"infer_order\":" << n.infer_order << ",\"arg\":[";
  for (size_t i = 0; i < n.arg.size(); ++i) {
    if (i) ss << ',';
    JsonArgument(ss, n.arg[i]);
  }
  ss << "],\"tensors\":[";
  for (size_t i = 0; i < n.tensors.size(); ++i) {
    const proto::ConstTensor &t = n.tensors[i];
    if (i) ss << ',';
    ss << "{\"name\":";
    JsonString(ss, t.name);
    ss << ",\"dims\":";
    JsonInts(ss, t.dims);
    ss << ",\"data_type\":" << t.data_type << ",\"float_data\":";
    JsonFloats(ss, t.float_data);
    ss << ",\"int32_data\":";
    JsonInts(ss, t.int32_data);
    ss << ",\"offset\":" << t.offset << ",\"data_size\":" << t.data_size << ",\"scale\":";
    JsonFloat(ss, t.scale);
    ss << ",\"zero_point\":" << t.zero_point << ",\"minval\":";
    JsonFloat(ss, t.minval);
    ss << ",\"maxval\":";
    JsonFloat(ss, t.maxval);
    ss << ",\"quantized\":" << (t.quantized ? "true" : "false") << ",\"node_id\":" << t.node_id << '}';
  }
  ss << "],\"op\":[";
  for (size_t i = 0; i < n.op.size(); ++i) {
    const proto::OperatorDef &o = n.op[i];
    if (i) ss << ',';
    ss << "{\"name\":";
    JsonString(ss, o.name);
    ss << ",\"type\":";
    JsonString(ss, o.type);
    ss << ",\"input\":";
    JsonStrings(ss, o.input);
    ss << ",\"output\":";
    JsonStrings(ss, o.output);
    ss << ",\"device_type\":" << o.device_type << ",\"arg\":[";
    for (size_t k = 0; k < o.arg.size(); ++k) {
      if (k) ss << ',';
      JsonArgument(ss, o.arg[k]);
    }
    ss << "],\"output_shape\":[";
    for (size_t k = 0; k < o.output_shape.size(); ++k) {
      if (k) ss << ',';
      JsonInts(ss, o.output_shape[k].dims);
    }
    ss << "],\"output_type\":";
    JsonInts(ss, o.output_type);
    ss << ",\"quantize_info\":[";
    for (size_t k = 0; k < o.quantize_info.size(); ++k) {
      const proto::QuantizeActivationInfo &q = o.quantize_info[k];
      if (k) ss << ',';
      ss << "{\"scale\":";
      JsonFloat(ss, q.scale);
      ss << ",\"zero_point\":" << q.zero_point << ",\"minval\":";
      JsonFloat(ss, q.minval);
      ss << ",\"maxval\":";
      JsonFloat(ss, q.maxval);
      ss << '}';
    }
    ss << "],\"mem_id\":";
    JsonInts(ss, o.mem_id);
    ss << ",\"node_id\":" << o.node_id << ",\"op_id\":" << o.op_id << ",\"padding\":" << o.padding
       << ",\"node_input\":[";
    for (size_t k = 0; k < o.node_input.size(); ++k)
      ss << (k ? "," : "") << '[' << o.node_input[k].node_id << ',' << o.node_input[k].output_port << ']';
    ss << "],\"out_max_byte_size\":";
    JsonInts(ss, o.out_max_byte_size);
    ss << '}';
  }
  ss << "],\"input_info\":[";
  for (size_t i = 0; i < n.input_info.size(); ++i) {
    if (i) ss << ',';
    JsonInfo(ss, n.input_info[i]);
  }
  ss << "],\"output_info\":[";
  for (size_t i = 0; i < n.output_info.size(); ++i) {
    if (i) ss << ',';
    JsonInfo(ss, n.output_info[i]);
  }
  ss << "]}";
  return ss.str();
}

int GetNetArgInt(const proto::NetDef &net_def, const std::string &name, int default_value) {
  // a later argument of the same name replaces an earlier one, as in the helper's map
  int value = default_value;
  for (const proto::Argument &a : net_def.arg)
    if (a.name == name && a.has_i) value = static_cast<int>(a.i);
  return value;
}

void ConvertOperatorDef(const proto::OperatorDef &src, OperatorDef *dst) {
  *dst = OperatorDef();
  dst->type = src.type;
  dst->name = src.name;
  dst->input = src.input;
  dst->output = src.output;
  for (const proto::Argument &a : src.arg) {
    if (a.has_i) dst->i[a.name] = static_cast<int>(a.i);
    if (a.has_f) dst->f[a.name] = a.f;
    if (a.has_s) dst->s[a.name] = a.s;
    if (!a.ints.empty()) dst->ints[a.name] = std::vector<int>(a.ints.begin(), a.ints.end());
    if (!a.floats.empty()) dst->floats[a.name] = a.floats;
  }
  for (int t : src.output_type) dst->output_type.push_back(static_cast<DataType>(t));
  for (const proto::QuantizeActivationInfo &q : src.quantize_info) {
    QuantizeActivationInfo info;
    info.scale = q.scale;
    info.zero_point = q.zero_point;
    info.minval = q.minval;
    info.maxval = q.maxval;
    dst->quantize_info.push_back(info);
  }
}

float HalfToFloat(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal half: normalise
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while ((man & 0x400u) == 0);
      bits = sign | static_cast<uint32_t>(127 - 15 - e) << 23 | (man & 0x3ffu) << 13;
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | man << 13;
  } else {
    bits = sign | (exp + 127 - 15) << 23 | man << 13;
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

}  // namespace mace
