// Reader for the reference's protobuf binary models (`.shadowmodel`): a decoder of the protobuf
// wire format for the five messages of shadow/proto/shadow.proto:5-47 (Blob, Argument, OpParam,
// NetParam, MetaNetParam), written against the wire-format specification - no protobuf runtime
// is linked.  Entry points mirror shadow/util/io.hpp:20-27 (ReadProtoFromArray,
// ReadProtoFromBinaryFile) for the two top-level messages.
//
// Wire format in short: a message is a sequence of (tag, value); tag = field_number << 3 | type;
// type 0 = varint, 1 = 64-bit, 2 = length-delimited (strings, bytes, nested messages, packed
// repeated scalars), 5 = 32-bit.  Repeated scalars are accepted packed and unpacked, whatever
// the schema declares, as the specification requires of a parser.  Unknown fields are skipped.
// int32 values travel as (sign-extended, up to 10-byte) varints.
#include <cstring>
#include <fstream>
#include <sstream>

#include "shadow_api.hpp"

namespace Shadow {
namespace {

class Reader {
 public:
  Reader(const unsigned char* p, size_t n) : p_(p), end_(p + n) {}
  bool done() const { return p_ >= end_; }

  uint64_t varint() {
    uint64_t v = 0;
    for (int shift = 0; shift < 64; shift += 7) {
      CHECK(p_ < end_) << "protobuf: truncated varint";
      const unsigned char b = *p_++;
      v |= static_cast<uint64_t>(b & 0x7f) << shift;
      if (!(b & 0x80)) return v;
    }
    LOG(FATAL) << "protobuf: varint longer than 10 bytes";
    return 0;
  }
  uint32_t fixed32() {
    CHECK(end_ - p_ >= 4) << "protobuf: truncated 32-bit value";
    uint32_t v;
    std::memcpy(&v, p_, 4);   // little-endian host (x86-64, aarch64)
    p_ += 4;
    return v;
  }
  Reader sub() {   // a length-delimited payload
    const uint64_t n = varint();
    CHECK(n <= static_cast<uint64_t>(end_ - p_)) << "protobuf: length runs past the end of the buffer";
    Reader r(p_, static_cast<size_t>(n));
    p_ += n;
    return r;
  }
  std::string str() {
    Reader r = sub();
    return std::string(reinterpret_cast<const char*>(r.p_), static_cast<size_t>(r.end_ - r.p_));
  }
  size_t remaining() const { return static_cast<size_t>(end_ - p_); }
  void skip(int wire_type) {
    switch (wire_type) {
      case 0: varint(); break;
      case 1: CHECK(end_ - p_ >= 8) << "protobuf: truncated 64-bit value"; p_ += 8; break;
      case 2: sub(); break;
      case 5: fixed32(); break;
      default: LOG(FATAL) << "protobuf: unsupported wire type " << wire_type;
    }
  }

 private:
  const unsigned char* p_;
  const unsigned char* end_;
};

float as_float(uint32_t bits) {
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}
int as_int32(uint64_t v) { return static_cast<int>(static_cast<int64_t>(v)); }

// repeated float / int32, packed (wire type 2) or one value per tag
template <typename Add>
void repeated_float(Reader& r, int wire_type, Add add) {
  if (wire_type == 2) {
    Reader p = r.sub();
    CHECK(p.remaining() % 4 == 0) << "protobuf: packed float payload is not a multiple of 4 bytes";
    while (!p.done()) add(as_float(p.fixed32()));
  } else {
    CHECK_EQ(wire_type, 5);
    add(as_float(r.fixed32()));
  }
}
template <typename Add>
void repeated_int32(Reader& r, int wire_type, Add add) {
  if (wire_type == 2) {
    Reader p = r.sub();
    while (!p.done()) add(as_int32(p.varint()));
  } else {
    CHECK_EQ(wire_type, 0);
    add(as_int32(r.varint()));
  }
}

void parse_blob(Reader r, shadow::Blob* blob) {
  while (!r.done()) {
    const uint64_t tag = r.varint();
    const int field = static_cast<int>(tag >> 3), wt = static_cast<int>(tag & 7);
    switch (field) {
      case 1: CHECK_EQ(wt, 2); blob->set_name(r.str()); break;
      case 2: CHECK_EQ(wt, 2); blob->set_type(r.str()); break;
      case 3: repeated_int32(r, wt, [&](int v) { blob->add_shape(v); }); break;
      case 4: repeated_float(r, wt, [&](float v) { blob->add_data_f(v); }); break;
      case 5: repeated_int32(r, wt, [&](int v) { blob->add_data_i(v); }); break;
      case 6: {
        CHECK_EQ(wt, 2);
        const std::string bytes = r.str();
        blob->add_data_b(std::vector<char>(bytes.begin(), bytes.end()));
        break;
      }
      default: r.skip(wt);
    }
  }
}

void parse_argument(Reader r, shadow::Argument* arg) {
  while (!r.done()) {
    const uint64_t tag = r.varint();
    const int field = static_cast<int>(tag >> 3), wt = static_cast<int>(tag & 7);
    switch (field) {
      case 1: CHECK_EQ(wt, 2); arg->set_name(r.str()); break;
      case 2: CHECK_EQ(wt, 5); arg->set_s_f(as_float(r.fixed32())); break;
      case 3: CHECK_EQ(wt, 0); arg->set_s_i(as_int32(r.varint())); break;
      case 4: CHECK_EQ(wt, 2); arg->set_s_s(r.str()); break;
      case 5: repeated_float(r, wt, [&](float v) { arg->add_v_f(v); }); break;
      case 6: repeated_int32(r, wt, [&](int v) { arg->add_v_i(v); }); break;
      case 7: CHECK_EQ(wt, 2); arg->add_v_s(r.str()); break;
      default: r.skip(wt);
    }
  }
}

void parse_op(Reader r, shadow::OpParam* op) {
  while (!r.done()) {
    const uint64_t tag = r.varint();
    const int field = static_cast<int>(tag >> 3), wt = static_cast<int>(tag & 7);
    switch (field) {
      case 1: CHECK_EQ(wt, 2); op->set_name(r.str()); break;
      case 2: CHECK_EQ(wt, 2); op->set_type(r.str()); break;
      case 3: CHECK_EQ(wt, 2); op->add_bottom(r.str()); break;
      case 4: CHECK_EQ(wt, 2); op->add_top(r.str()); break;
      case 11: CHECK_EQ(wt, 2); parse_argument(r.sub(), op->add_arg()); break;
      default: r.skip(wt);
    }
  }
}

void parse_net(Reader r, shadow::NetParam* net) {
  while (!r.done()) {
    const uint64_t tag = r.varint();
    const int field = static_cast<int>(tag >> 3), wt = static_cast<int>(tag & 7);
    switch (field) {
      case 1: CHECK_EQ(wt, 2); net->set_name(r.str()); break;
      case 5: CHECK_EQ(wt, 2); parse_blob(r.sub(), net->add_blob()); break;
      case 11: CHECK_EQ(wt, 2); parse_op(r.sub(), net->add_op()); break;
      case 12: CHECK_EQ(wt, 2); parse_argument(r.sub(), net->add_arg()); break;
      default: r.skip(wt);
    }
  }
}

void parse_meta(Reader r, shadow::MetaNetParam* meta) {
  while (!r.done()) {
    const uint64_t tag = r.varint();
    const int field = static_cast<int>(tag >> 3), wt = static_cast<int>(tag & 7);
    switch (field) {
      case 1: CHECK_EQ(wt, 2); meta->set_name(r.str()); break;
      case 11: CHECK_EQ(wt, 2); parse_net(r.sub(), meta->add_network()); break;
      case 12: CHECK_EQ(wt, 2); parse_argument(r.sub(), meta->add_arg()); break;
      default: r.skip(wt);
    }
  }
}

bool read_file(const std::string& path, std::string* bytes) {
  std::ifstream file(path, std::ios::binary);
  if (!file.is_open()) return false;
  std::stringstream ss;
  ss << file.rdbuf();
  *bytes = ss.str();
  return true;
}

}  // namespace

namespace IO {

bool ReadProtoFromArray(const void* proto_data, int proto_size, shadow::NetParam* proto) {
  CHECK_NOTNULL(proto);
  CHECK(proto_data != nullptr && proto_size >= 0);
  *proto = shadow::NetParam();
  parse_net(Reader(static_cast<const unsigned char*>(proto_data), static_cast<size_t>(proto_size)), proto);
  return true;
}

bool ReadProtoFromArray(const void* proto_data, int proto_size, shadow::MetaNetParam* proto) {
  CHECK_NOTNULL(proto);
  CHECK(proto_data != nullptr && proto_size >= 0);
  *proto = shadow::MetaNetParam();
  parse_meta(Reader(static_cast<const unsigned char*>(proto_data), static_cast<size_t>(proto_size)), proto);
  return true;
}

bool ReadProtoFromBinaryFile(const std::string& proto_file, shadow::NetParam* proto) {
  std::string bytes;
  if (!read_file(proto_file, &bytes)) return false;
  return ReadProtoFromArray(bytes.data(), static_cast<int>(bytes.size()), proto);
}

bool ReadProtoFromBinaryFile(const std::string& proto_file, shadow::MetaNetParam* proto) {
  std::string bytes;
  if (!read_file(proto_file, &bytes)) return false;
  return ReadProtoFromArray(bytes.data(), static_cast<int>(bytes.size()), proto);
}

}  // namespace IO
}  // namespace Shadow
