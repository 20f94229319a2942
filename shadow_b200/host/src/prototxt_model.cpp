// Reader for models in protobuf TEXT format (`.shadowtxt`: what TextFormat prints for the messages of
// shadow/proto/shadow.proto:5-47), written against the text-format grammar - no protobuf runtime is
// linked.  Supported: `field: value`, `field { ... }` and `field: { ... }` for messages (also with
// < >), `field: [v, v, ...]` for repeated scalars, quoted strings with C escapes and adjacent-string
// concatenation, `#` comments, optional `,` / `;` separators, decimal / hex / octal integers, floats
// with an optional `f` suffix, `inf` / `nan`.  Unknown field names are refused (as TextFormat does).
#include <cctype>
#include <cmath>
#include <cstdlib>

#include "shadow_api.hpp"

namespace Shadow {
namespace {

class Lexer {
 public:
  explicit Lexer(const std::string& s) : s_(s) {}

  void skip_space() {
    while (pos_ < s_.size()) {
      const char c = s_[pos_];
      if (c == '#') {
        while (pos_ < s_.size() && s_[pos_] != '\n') ++pos_;
      } else if (std::isspace(static_cast<unsigned char>(c))) {
        ++pos_;
      } else {
        break;
      }
    }
  }
  bool at_end() { skip_space(); return pos_ >= s_.size(); }
  char peek() { skip_space(); return pos_ < s_.size() ? s_[pos_] : '\0'; }
  bool accept(char c) {
    if (peek() == c) { ++pos_; return true; }
    return false;
  }
  void expect(char c) { CHECK(accept(c)) << "model text: expected '" << c << "' near offset " << pos_; }

  std::string identifier() {
    skip_space();
    const size_t b = pos_;
    while (pos_ < s_.size() && (std::isalnum(static_cast<unsigned char>(s_[pos_])) || s_[pos_] == '_')) ++pos_;
    CHECK(pos_ > b) << "model text: expected a field name near offset " << b;
    return s_.substr(b, pos_ - b);
  }

  // a number / identifier-like scalar token (no quotes)
  std::string scalar() {
    skip_space();
    const size_t b = pos_;
    while (pos_ < s_.size()) {
      const char c = s_[pos_];
      if (std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '.' || c == '+' || c == '-') ++pos_;
      else break;
    }
    CHECK(pos_ > b) << "model text: expected a value near offset " << b;
    return s_.substr(b, pos_ - b);
  }

  // one or more adjacent quoted strings, concatenated
  std::string quoted() {
    std::string out;
    CHECK(peek() == '"' || peek() == '\'') << "model text: expected a quoted string near offset " << pos_;
    while (peek() == '"' || peek() == '\'') {
      const char q = s_[pos_++];
      while (true) {
        CHECK(pos_ < s_.size()) << "model text: unterminated string";
        char c = s_[pos_++];
        if (c == q) break;
        if (c != '\\') { out.push_back(c); continue; }
        CHECK(pos_ < s_.size()) << "model text: unterminated escape";
        c = s_[pos_++];
        switch (c) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'r': out.push_back('\r'); break;
          case 'a': out.push_back('\a'); break;
          case 'b': out.push_back('\b'); break;
          case 'f': out.push_back('\f'); break;
          case 'v': out.push_back('\v'); break;
          case '\\': case '\'': case '"': case '?': out.push_back(c); break;
          case 'x': case 'X': {
            int v = 0, n = 0;
            while (n < 2 && pos_ < s_.size() && std::isxdigit(static_cast<unsigned char>(s_[pos_]))) {
              const char h = s_[pos_++];
              v = v * 16 + (std::isdigit(static_cast<unsigned char>(h)) ? h - '0' : (std::tolower(h) - 'a' + 10));
              ++n;
            }
            CHECK(n > 0) << "model text: \\x without hex digits";
            out.push_back(static_cast<char>(v));
            break;
          }
          default: {
            CHECK(c >= '0' && c <= '7') << "model text: unknown escape \\" << c;
            int v = c - '0', n = 1;
            while (n < 3 && pos_ < s_.size() && s_[pos_] >= '0' && s_[pos_] <= '7') { v = v * 8 + (s_[pos_++] - '0'); ++n; }
            out.push_back(static_cast<char>(v));
          }
        }
      }
    }
    return out;
  }

 private:
  const std::string& s_;
  size_t pos_ = 0;
};

int to_int(const std::string& t) {
  char* end = nullptr;
  const long long v = std::strtoll(t.c_str(), &end, 0);   // base 0: decimal, 0x hex, 0 octal
  CHECK(end != nullptr && *end == '\0') << "model text: '" << t << "' is not an integer";
  CHECK(v >= -2147483648ll && v <= 2147483647ll) << "model text: " << t << " does not fit int32";
  return static_cast<int>(v);
}

float to_float(std::string t) {
  std::string low;
  for (char c : t) low.push_back(static_cast<char>(std::tolower(static_cast<unsigned char>(c))));
  if (low == "inf" || low == "+inf" || low == "infinity") return INFINITY;
  if (low == "-inf" || low == "-infinity") return -INFINITY;
  if (low == "nan" || low == "-nan") return NAN;
  if (!t.empty() && (t.back() == 'f' || t.back() == 'F')) t.pop_back();
  char* end = nullptr;
  const float v = std::strtof(t.c_str(), &end);
  CHECK(end != nullptr && *end == '\0' && !t.empty()) << "model text: '" << t << "' is not a number";
  return v;
}

// `: v` or `: [v, v]` for a scalar field; calls add(token-reader) once per value
template <typename One>
void scalar_values(Lexer& lx, One one) {
  lx.expect(':');
  if (lx.accept('[')) {
    if (lx.accept(']')) return;
    do { one(); } while (lx.accept(','));
    lx.expect(']');
  } else {
    one();
  }
}

// `{ ... }`, `: { ... }`, `< ... >`: parses the body with `body(lexer, closing char)`
template <typename Body>
void message_value(Lexer& lx, Body body) {
  lx.accept(':');
  char close = '}';
  if (lx.accept('<')) close = '>';
  else lx.expect('{');
  body(close);
}

void separators(Lexer& lx) { while (lx.accept(',') || lx.accept(';')) {} }

void parse_blob(Lexer& lx, char close, shadow::Blob* b) {
  while (!lx.accept(close)) {
    const std::string f = lx.identifier();
    if (f == "name") scalar_values(lx, [&] { b->set_name(lx.quoted()); });
    else if (f == "type") scalar_values(lx, [&] { b->set_type(lx.quoted()); });
    else if (f == "shape") scalar_values(lx, [&] { b->add_shape(to_int(lx.scalar())); });
    else if (f == "data_f") scalar_values(lx, [&] { b->add_data_f(to_float(lx.scalar())); });
    else if (f == "data_i") scalar_values(lx, [&] { b->add_data_i(to_int(lx.scalar())); });
    else if (f == "data_b") scalar_values(lx, [&] { const std::string s = lx.quoted(); b->add_data_b(std::vector<char>(s.begin(), s.end())); });
    else LOG(FATAL) << "model text: Blob has no field '" << f << "'";
    separators(lx);
  }
}

void parse_argument(Lexer& lx, char close, shadow::Argument* a) {
  while (!lx.accept(close)) {
    const std::string f = lx.identifier();
    if (f == "name") scalar_values(lx, [&] { a->set_name(lx.quoted()); });
    else if (f == "s_f") scalar_values(lx, [&] { a->set_s_f(to_float(lx.scalar())); });
    else if (f == "s_i") scalar_values(lx, [&] { a->set_s_i(to_int(lx.scalar())); });
    else if (f == "s_s") scalar_values(lx, [&] { a->set_s_s(lx.quoted()); });
    else if (f == "v_f") scalar_values(lx, [&] { a->add_v_f(to_float(lx.scalar())); });
    else if (f == "v_i") scalar_values(lx, [&] { a->add_v_i(to_int(lx.scalar())); });
    else if (f == "v_s") scalar_values(lx, [&] { a->add_v_s(lx.quoted()); });
    else LOG(FATAL) << "model text: Argument has no field '" << f << "'";
    separators(lx);
  }
}

void parse_op(Lexer& lx, char close, shadow::OpParam* op) {
  while (!lx.accept(close)) {
    const std::string f = lx.identifier();
    if (f == "name") scalar_values(lx, [&] { op->set_name(lx.quoted()); });
    else if (f == "type") scalar_values(lx, [&] { op->set_type(lx.quoted()); });
    else if (f == "bottom") scalar_values(lx, [&] { op->add_bottom(lx.quoted()); });
    else if (f == "top") scalar_values(lx, [&] { op->add_top(lx.quoted()); });
    else if (f == "arg") message_value(lx, [&](char c) { parse_argument(lx, c, op->add_arg()); });
    else LOG(FATAL) << "model text: OpParam has no field '" << f << "'";
    separators(lx);
  }
}

// close == '\0': top level, ends with the input
void parse_net(Lexer& lx, char close, shadow::NetParam* net) {
  while (close == '\0' ? !lx.at_end() : !lx.accept(close)) {
    const std::string f = lx.identifier();
    if (f == "name") scalar_values(lx, [&] { net->set_name(lx.quoted()); });
    else if (f == "blob") message_value(lx, [&](char c) { parse_blob(lx, c, net->add_blob()); });
    else if (f == "op") message_value(lx, [&](char c) { parse_op(lx, c, net->add_op()); });
    else if (f == "arg") message_value(lx, [&](char c) { parse_argument(lx, c, net->add_arg()); });
    else LOG(FATAL) << "model text: NetParam has no field '" << f << "'";
    separators(lx);
  }
}

void parse_meta(Lexer& lx, shadow::MetaNetParam* meta) {
  while (!lx.at_end()) {
    const std::string f = lx.identifier();
    if (f == "name") scalar_values(lx, [&] { meta->set_name(lx.quoted()); });
    else if (f == "network") message_value(lx, [&](char c) { parse_net(lx, c, meta->add_network()); });
    else if (f == "arg") message_value(lx, [&](char c) { parse_argument(lx, c, meta->add_arg()); });
    else LOG(FATAL) << "model text: MetaNetParam has no field '" << f << "'";
    separators(lx);
  }
}

}  // namespace

namespace IO {

bool ReadProtoFromProtoText(const std::string& proto_text, shadow::NetParam* proto) {
  CHECK_NOTNULL(proto);
  *proto = shadow::NetParam();
  Lexer lx(proto_text);
  parse_net(lx, '\0', proto);
  return true;
}

bool ReadProtoFromProtoText(const std::string& proto_text, shadow::MetaNetParam* proto) {
  CHECK_NOTNULL(proto);
  *proto = shadow::MetaNetParam();
  Lexer lx(proto_text);
  parse_meta(lx, proto);
  return true;
}

}  // namespace IO
}  // namespace Shadow
