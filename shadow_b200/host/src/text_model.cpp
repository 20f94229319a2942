// Reader for the reference's protobuf-free text model format (shadow/core/parser.cpp:1034-1917,
// entered through IO::ReadProtoFromText, shadow/util/io.cpp):
//
//   line 1   [net name]
//   line 2   [{arg, type, [v # v]}; ...]                 network arguments
//   line 3   [{blob, type, [d # d]}; ...]                weight blobs
//   line 4+  [Type] | [name] | [nBottom nTop nArg] | [bottoms; ...] | [tops; ...] | [{arg, type, [v]}; ...]
//
// with type one of s_f, s_i, s_s, v_f, v_i, v_s.  Like the reference, an operator line keeps only
// the arguments its type knows and fills the others in with the parser's defaults - which are not
// always the operator's own defaults (Scale: has_scale/has_bias default to 1 here, 0 in the
// operator) - so the table below states them per type.  Operator types outside this library's
// scope are refused at parse time.
#include <cstdlib>
#include <fstream>
#include <map>
#include <sstream>

#include "shadow_api.hpp"

namespace Shadow {
namespace {

std::string trim(const std::string& s) {
  const auto b = s.find_first_not_of(" \t\r\n");
  if (b == std::string::npos) return "";
  const auto e = s.find_last_not_of(" \t\r\n");
  return s.substr(b, e - b + 1);
}

// pieces between delimiters, empty pieces dropped (the reference's Util::tokenize)
std::vector<std::string> tokenize(const std::string& s, char delim) {
  std::vector<std::string> out;
  std::string cur;
  for (char c : s) {
    if (c == delim) {
      if (!cur.empty()) out.push_back(cur);
      cur.clear();
    } else {
      cur.push_back(c);
    }
  }
  if (!cur.empty()) out.push_back(cur);
  return out;
}

// "[...]" or "{...}" without its first and last character
std::string unwrap(const std::string& s) {
  CHECK_GE(s.size(), 2u) << "malformed model text near '" << s << "'";
  return s.substr(1, s.size() - 2);
}

struct Value {
  std::string type;
  float s_f = 0;
  int s_i = 0;
  std::string s_s;
  VecFloat v_f;
  VecInt v_i;
  VecString v_s;
};

// "{name, type, [value]}; {name, type, [value]}; ..."
std::map<std::string, Value> parse_arguments(const std::string& text) {
  std::map<std::string, Value> args;
  for (const auto& item : tokenize(text, ';')) {
    const auto parts = tokenize(unwrap(trim(item)), ',');
    CHECK_EQ(parts.size(), 3u);
    const std::string name = trim(parts[0]), type = trim(parts[1]), value = unwrap(trim(parts[2]));
    Value v;
    v.type = type;
    if (type == "s_f") v.s_f = std::strtof(value.c_str(), nullptr);
    else if (type == "s_i") v.s_i = static_cast<int>(std::strtol(value.c_str(), nullptr, 10));
    else if (type == "s_s") v.s_s = value;
    else if (type == "v_f") { for (const auto& t : tokenize(value, '#')) v.v_f.push_back(std::strtof(trim(t).c_str(), nullptr)); }
    else if (type == "v_i") { for (const auto& t : tokenize(value, '#')) v.v_i.push_back(static_cast<int>(std::strtol(trim(t).c_str(), nullptr, 10))); }
    else if (type == "v_s") { for (const auto& t : tokenize(value, '#')) v.v_s.push_back(trim(t)); }
    else LOG(FATAL) << "Unsupported argument type " << type;
    args[name] = v;
  }
  return args;
}

void put(shadow::OpParam* op, const std::string& name, int v) { auto* a = op->add_arg(); a->set_name(name); a->set_s_i(v); }
void put(shadow::OpParam* op, const std::string& name, float v) { auto* a = op->add_arg(); a->set_name(name); a->set_s_f(v); }
void put(shadow::OpParam* op, const std::string& name, const VecInt& v) {
  auto* a = op->add_arg();
  a->set_name(name);
  for (int x : v) a->add_v_i(x);
}
void put(shadow::OpParam* op, const std::string& name, const VecFloat& v) {
  auto* a = op->add_arg();
  a->set_name(name);
  for (float x : v) a->add_v_f(x);
}

// What the parser emits for one argument of one operator type.
enum Kind { kInt, kFloat, kInts, kFloats };
struct Spec {
  const char* name;
  Kind kind;
  double fallback;     // kInt / kFloat: emitted when the line does not give the argument
  bool only_if_given;  // emitted only when the line gives it (Binary's scalar)
};

// Operator types of this library that the text format knows, in the reference's lookup order
// (the first entry whose name occurs INSIDE the type string wins, shadow/core/parser.cpp:1901-1908).
const std::vector<std::pair<std::string, std::vector<Spec>>>& op_table() {
  static const std::vector<std::pair<std::string, std::vector<Spec>>> table = {
      {"Activate", {{"type", kInt, 1, false}, {"slope", kFloat, 0.1, false}}},
      {"BatchNorm", {{"use_global_stats", kInt, 1, false}, {"eps", kFloat, 1e-5, false}}},
      {"Binary", {{"operation", kInt, -1, false}, {"scalar", kFloat, 0, true}}},
      {"Concat", {{"axis", kInt, 1, false}}},
      {"Eltwise", {{"operation", kInt, 1, false}, {"coeff", kFloats, 0, false}}},
      {"Flatten", {{"axis", kInt, 1, false}, {"end_axis", kInt, -1, false}}},
      {"Gather", {{"axis", kInt, 0, false}, {"indexes", kInts, 0, false}}},
      {"Input", {}},   // every argument is a top's shape (v_i), forwarded as it is
      {"InstanceNorm", {{"eps", kFloat, 1e-5, false}}},
      {"Pad", {{"paddings", kInts, 0, false}, {"value", kFloat, 0, false}}},
      {"Permute", {{"order", kInts, 0, false}}},
      {"Pooling", {{"pool", kInt, 0, false}, {"kernel_size", kInts, 0, false}, {"stride", kInts, 0, false},
                   {"pad", kInts, 0, false}, {"global_pooling", kInt, 0, false}, {"full_pooling", kInt, 1, false}}},
      {"Reduce", {{"operation", kInt, 0, false}, {"axes", kInts, 0, false}, {"keep_dims", kInt, 1, false}}},
      {"Reshape", {{"shape", kInts, 0, false}, {"axis", kInt, 0, false}, {"num_axes", kInt, -1, false}}},
      {"Scale", {{"axis", kInt, 1, false}, {"has_scale", kInt, 1, false}, {"has_bias", kInt, 1, false},
                 {"scale_value", kFloats, 0, false}, {"bias_value", kFloats, 0, false}}},
      {"Slice", {{"axis", kInt, 1, false}, {"slice_point", kInts, 0, false}}},
      {"Softmax", {{"axis", kInt, 1, false}}},
      {"Squeeze", {{"axes", kInts, 0, false}}},
      {"SSDNormalize", {{"across_spatial", kInt, 1, false}, {"channel_shared", kInt, 1, false}}},
      {"Stack", {{"axis", kInt, 0, false}}},
      {"Unary", {{"operation", kInt, -1, false}}},
      {"Unsqueeze", {{"axes", kInts, 0, false}}},
  };
  return table;
}

shadow::OpParam parse_op(const std::vector<std::string>& fields, const std::string& table_name, const std::vector<Spec>& specs) {
  shadow::OpParam op;
  op.set_type(fields[0]);
  op.set_name(fields[1]);
  const auto counts = tokenize(fields[2], ' ');
  CHECK_EQ(counts.size(), 3u);
  if (std::atoi(counts[0].c_str()) > 0)
    for (const auto& b : tokenize(fields[3], ';')) op.add_bottom(trim(b));
  if (std::atoi(counts[1].c_str()) > 0)
    for (const auto& t : tokenize(fields[4], ';')) op.add_top(trim(t));
  std::map<std::string, Value> given;
  if (std::atoi(counts[2].c_str()) > 0) given = parse_arguments(fields[5]);
  if (table_name == "Input") {
    for (const auto& kv : given) put(&op, kv.first, kv.second.v_i);
    return op;
  }
  for (const auto& spec : specs) {
    const auto it = given.find(spec.name);
    const bool has = it != given.end();
    if (spec.only_if_given && !has) continue;
    switch (spec.kind) {
      case kInt: put(&op, spec.name, has ? it->second.s_i : static_cast<int>(spec.fallback)); break;
      case kFloat: put(&op, spec.name, has ? it->second.s_f : static_cast<float>(spec.fallback)); break;
      case kInts: put(&op, spec.name, has ? it->second.v_i : VecInt()); break;
      case kFloats: put(&op, spec.name, has ? it->second.v_f : VecFloat()); break;
    }
  }
  return op;
}

void parse_net(const std::string& text, shadow::NetParam* net) {
  const auto lines = tokenize(text, '\n');
  CHECK_GE(lines.size(), 3u) << "a text model has at least a name line, an argument line and a blob line";
  net->set_name(unwrap(trim(lines[0])));
  for (const auto& kv : parse_arguments(unwrap(trim(lines[1])))) {
    auto* a = net->add_arg();
    a->set_name(kv.first);
    const Value& v = kv.second;
    if (v.type == "s_f") a->set_s_f(v.s_f);
    else if (v.type == "s_i") a->set_s_i(v.s_i);
    else if (v.type == "s_s") a->set_s_s(v.s_s);
    else if (v.type == "v_f") { for (float x : v.v_f) a->add_v_f(x); }
    else if (v.type == "v_i") { for (int x : v.v_i) a->add_v_i(x); }
    else { for (const auto& x : v.v_s) a->add_v_s(x); }
  }
  for (const auto& item : tokenize(unwrap(trim(lines[2])), ';')) {
    const auto parts = tokenize(unwrap(trim(item)), ',');
    CHECK_EQ(parts.size(), 3u);
    auto* blob = net->add_blob();
    blob->set_name(trim(parts[0]));
    blob->set_type(trim(parts[1]));
    for (const auto& d : tokenize(unwrap(trim(parts[2])), '#')) blob->add_shape(std::atoi(trim(d).c_str()));
  }
  for (size_t i = 3; i < lines.size(); ++i) {
    if (trim(lines[i]).empty()) continue;
    auto fields = tokenize(lines[i], '|');
    CHECK_EQ(fields.size(), 6u);
    for (auto& f : fields) f = unwrap(trim(f));
    bool found = false;
    for (const auto& entry : op_table()) {
      if (fields[0].find(entry.first) != std::string::npos) {
        net->add_op(parse_op(fields, entry.first, entry.second));
        found = true;
        break;
      }
    }
    CHECK(found) << "Error when parsing op: " << fields[1] << ", op type: " << fields[0] << " is not recognized!";
  }
}

}  // namespace

namespace IO {

bool ReadProtoFromText(const std::string& proto_text, shadow::NetParam* proto) {
  CHECK_NOTNULL(proto);
  // the line-based format opens with "[net name]"; protobuf text format opens with a field name
  const auto first = proto_text.find_first_not_of(" \t\r\n");
  if (first != std::string::npos && proto_text[first] != '[') return ReadProtoFromProtoText(proto_text, proto);
  *proto = shadow::NetParam();
  parse_net(proto_text, proto);
  return true;
}

bool ReadProtoFromTextFile(const std::string& proto_file, shadow::NetParam* proto) {
  std::ifstream file(proto_file);
  if (!file.is_open()) return false;
  std::stringstream ss;
  ss << file.rdbuf();
  return ReadProtoFromText(ss.str(), proto);
}

}  // namespace IO
}  // namespace Shadow
