// NetDef readers: protobuf text format and protobuf wire format, written against
// the message definitions in blaze/blaze/proto/blaze.proto:22-115 (field numbers
// below) without a protobuf dependency.
#include <cctype>
#include <cmath>
#include <cstring>

#include "runtime.h"

namespace blaze {

// ---- text format --------------------------------------------------------------------------------
namespace {

struct Lexer {
  const std::string& s;
  size_t pos = 0;
  explicit Lexer(const std::string& text) : s(text) {}
  void SkipSpace() {
    while (pos < s.size()) {
      if (std::isspace((unsigned char)s[pos]) || s[pos] == ',' || s[pos] == ';') ++pos;
      else if (s[pos] == '#') { while (pos < s.size() && s[pos] != '\n') ++pos; }
      else break;
    }
  }
  bool AtEnd() { SkipSpace(); return pos >= s.size(); }
  char Peek() { SkipSpace(); return pos < s.size() ? s[pos] : 0; }
  // identifier or bare scalar
  std::string Word() {
    SkipSpace();
    size_t b = pos;
    while (pos < s.size() && !std::isspace((unsigned char)s[pos]) && !strchr("{}:,;#\"'<>", s[pos])) ++pos;
    return s.substr(b, pos - b);
  }
  bool String(std::string* out, std::string* err) {
    SkipSpace();
    const char quote = s[pos++];
    std::string r;
    while (pos < s.size() && s[pos] != quote) {
      char c = s[pos++];
      if (c == '\\' && pos < s.size()) {
        char e = s[pos++];
        switch (e) {
          case 'n': r += '\n'; break;
          case 't': r += '\t'; break;
          case 'r': r += '\r'; break;
          case '\\': r += '\\'; break;
          case '"': r += '"'; break;
          case '\'': r += '\''; break;
          default:
            if (e >= '0' && e <= '7') {            // octal escape
              int v = e - '0';
              for (int k = 0; k < 2 && pos < s.size() && s[pos] >= '0' && s[pos] <= '7'; ++k) v = v * 8 + (s[pos++] - '0');
              r += (char)v;
            } else r += e;
        }
      } else r += c;
    }
    if (pos >= s.size()) { *err = "unterminated string"; return false; }
    ++pos;
    *out = r;
    return true;
  }
};

bool ParseMessage(Lexer& lx, TextNode* node, bool top, std::string* err) {
  while (true) {
    if (lx.AtEnd()) {
      if (!top) { *err = "unexpected end of text inside a message"; return false; }
      return true;
    }
    char c = lx.Peek();
    if (c == '}' || c == '>') {
      if (top) { *err = "unbalanced closing brace"; return false; }
      ++lx.pos;
      return true;
    }
    std::string field = lx.Word();
    if (field.empty()) { *err = MakeString("expected a field name at offset ", lx.pos); return false; }
    if (lx.Peek() == ':') ++lx.pos;
    c = lx.Peek();
    if (c == '{' || c == '<') {
      ++lx.pos;
      std::unique_ptr<TextNode> child(new TextNode());
      if (!ParseMessage(lx, child.get(), false, err)) return false;
      node->children.emplace_back(field, std::move(child));
    } else if (c == '"' || c == '\'') {
      std::string v, more;
      if (!lx.String(&v, err)) return false;
      while (lx.Peek() == '"' || lx.Peek() == '\'') {       // adjacent string literals concatenate
        if (!lx.String(&more, err)) return false;
        v += more;
      }
      node->scalars.emplace(field, v);
    } else {
      std::string v = lx.Word();
      if (v.empty()) { *err = MakeString("expected a value for field ", field); return false; }
      node->scalars.emplace(field, v);
    }
  }
}

double ToDouble(const std::string& v) {
  std::string t = v;
  if (!t.empty() && (t.back() == 'f' || t.back() == 'F')) t.pop_back();   // text format allows 2.0f
  if (t == "inf" || t == "infinity") return INFINITY;
  if (t == "-inf" || t == "-infinity") return -INFINITY;
  if (t == "nan") return NAN;
  return std::strtod(t.c_str(), nullptr);
}
int64_t ToInt(const std::string& v) {
  if (v == "true") return 1;
  if (v == "false") return 0;
  if (v.find_first_of(".eE") != std::string::npos && v.find("0x") == std::string::npos) return (int64_t)ToDouble(v);
  return std::strtoll(v.c_str(), nullptr, 0);
}

void FillArgument(const TextNode& n, Argument* a) {
  std::string v;
  if (n.Get("name", &v)) a->name = v;
  if (n.Get("f", &v)) { a->has_f = true; a->f = (float)ToDouble(v); }
  if (n.Get("i", &v)) { a->has_i = true; a->i = ToInt(v); }
  if (n.Get("s", &v)) { a->has_s = true; a->s = v; }
  auto r = n.scalars.equal_range("floats");
  for (auto it = r.first; it != r.second; ++it) a->floats.push_back((float)ToDouble(it->second));
  r = n.scalars.equal_range("ints");
  for (auto it = r.first; it != r.second; ++it) a->ints.push_back(ToInt(it->second));
  r = n.scalars.equal_range("strings");
  for (auto it = r.first; it != r.second; ++it) a->strings.push_back(it->second);
}

void FillDevice(const TextNode& n, DeviceOption* d) {
  d->device_type = (int)n.GetInt("device_type", 0);
  d->device_id = (int)n.GetInt("device_id", 0);
  d->is_pipe = n.GetInt("is_pipe", 0) != 0;
}

void FillValueInfo(const TextNode& n, ValueInfo* v) {
  std::string s;
  if (n.Get("name", &s)) v->name = s;
  if (n.Get("feature_name", &s)) v->feature_name = s;
  if (n.Get("dtype", &s)) {
    if (s == "kFloat") v->dtype = kFloat; else if (s == "kFloat16") v->dtype = kFloat16;
    else if (s == "kInt32") v->dtype = kInt32; else if (s == "kInt64") v->dtype = kInt64;
    else v->dtype = (int)ToInt(s);
  }
  v->level = (int)n.GetInt("level", 0);
  v->input_type = (int)n.GetInt("input_type", 0);
}

}  // namespace

std::vector<const TextNode*> TextNode::Children(const std::string& name) const {
  std::vector<const TextNode*> out;
  for (const auto& c : children)
    if (c.first == name) out.push_back(c.second.get());
  return out;
}
bool TextNode::Get(const std::string& name, std::string* v) const {
  auto it = scalars.find(name);
  if (it == scalars.end()) return false;
  // multimap keeps insertion order for equal keys; the last value wins for a singular field
  auto r = scalars.equal_range(name);
  for (auto i = r.first; i != r.second; ++i) *v = i->second;
  return true;
}
int64_t TextNode::GetInt(const std::string& name, int64_t def) const {
  std::string v;
  return Get(name, &v) ? ToInt(v) : def;
}

bool ParseTextProto(const std::string& text, TextNode* root, std::string* err) {
  Lexer lx(text);
  return ParseMessage(lx, root, true, err);
}

bool ParseNetDefText(const std::string& text, NetDef* out, std::string* err) {
  TextNode root;
  if (!ParseTextProto(text, &root, err)) return false;
  std::string v;
  *out = NetDef();
  if (root.Get("name", &v)) out->name = v;
  if (root.Get("run_mode", &v)) out->run_mode = v;
  for (const auto& c : root.children) {
    const TextNode& n = *c.second;
    if (c.first == "op") {
      OperatorDef op;
      if (n.Get("type", &v)) op.type = v;
      if (n.Get("name", &v)) op.name = v;
      // repeated scalars keep their order inside the multimap's equal range
      auto r = n.scalars.equal_range("input");
      for (auto it = r.first; it != r.second; ++it) op.input.push_back(it->second);
      r = n.scalars.equal_range("output");
      for (auto it = r.first; it != r.second; ++it) op.output.push_back(it->second);
      for (const TextNode* a : n.Children("arg")) { op.arg.emplace_back(); FillArgument(*a, &op.arg.back()); }
      auto dev = n.Children("device_option");
      if (!dev.empty()) { op.has_device_option = true; FillDevice(*dev[0], &op.device_option); }
      if (op.type.empty()) { *err = "operator without a type"; return false; }
      out->op.push_back(op);
    } else if (c.first == "arg") {
      out->arg.emplace_back();
      FillArgument(n, &out->arg.back());
    } else if (c.first == "device_option") {
      FillDevice(n, &out->device_option);
    } else if (c.first == "external_input") {
      out->external_input.emplace_back();
      FillValueInfo(n, &out->external_input.back());
    } else if (c.first == "external_output") {
      out->external_output.emplace_back();
      FillValueInfo(n, &out->external_output.back());
    }
  }
  return true;
}

// ---- wire format --------------------------------------------------------------------------------
namespace {

struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  bool ok = true;
  uint64_t Varint() {
    uint64_t v = 0;
    int shift = 0;
    while (p < end && shift < 64) {
      uint8_t b = *p++;
      v |= (uint64_t)(b & 0x7f) << shift;
      if (!(b & 0x80)) return v;
      shift += 7;
    }
    ok = false;
    return 0;
  }
  Reader Sub() {
    uint64_t n = Varint();
    if (!ok || n > (uint64_t)(end - p)) { ok = false; return Reader{p, p}; }
    Reader r{p, p + n};
    p += n;
    return r;
  }
  std::string Bytes() {
    Reader r = Sub();
    return std::string(reinterpret_cast<const char*>(r.p), r.end - r.p);
  }
  float Fixed32() {
    if (end - p < 4) { ok = false; return 0; }
    float f;
    memcpy(&f, p, 4);
    p += 4;
    return f;
  }
  void Skip(int wire) {
    switch (wire) {
      case 0: Varint(); break;
      case 1: if (end - p >= 8) p += 8; else ok = false; break;
      case 2: Sub(); break;
      case 5: if (end - p >= 4) p += 4; else ok = false; break;
      default: ok = false;
    }
  }
};

bool ReadArgument(Reader r, Argument* a) {
  while (r.ok && r.p < r.end) {
    uint64_t tag = r.Varint();
    int field = (int)(tag >> 3), wire = (int)(tag & 7);
    if (field == 1 && wire == 2) a->name = r.Bytes();
    else if (field == 2 && wire == 5) { a->has_f = true; a->f = r.Fixed32(); }
    else if (field == 3 && wire == 0) { a->has_i = true; a->i = (int64_t)r.Varint(); }
    else if (field == 4 && wire == 2) { a->has_s = true; a->s = r.Bytes(); }
    else if (field == 5 && wire == 2) { Reader s = r.Sub(); while (s.ok && s.p < s.end) a->floats.push_back(s.Fixed32()); }
    else if (field == 5 && wire == 5) a->floats.push_back(r.Fixed32());
    else if (field == 6 && wire == 2) { Reader s = r.Sub(); while (s.ok && s.p < s.end) a->ints.push_back((int64_t)s.Varint()); }
    else if (field == 6 && wire == 0) a->ints.push_back((int64_t)r.Varint());
    else if (field == 7 && wire == 2) a->strings.push_back(r.Bytes());
    else r.Skip(wire);
  }
  return r.ok;
}

bool ReadDevice(Reader r, DeviceOption* d) {
  while (r.ok && r.p < r.end) {
    uint64_t tag = r.Varint();
    int field = (int)(tag >> 3), wire = (int)(tag & 7);
    if (field == 1 && wire == 0) d->device_type = (int)r.Varint();
    else if (field == 2 && wire == 0) d->device_id = (int)r.Varint();
    else if (field == 3 && wire == 0) d->is_pipe = r.Varint() != 0;
    else r.Skip(wire);
  }
  return r.ok;
}

bool ReadOperator(Reader r, OperatorDef* op) {
  while (r.ok && r.p < r.end) {
    uint64_t tag = r.Varint();
    int field = (int)(tag >> 3), wire = (int)(tag & 7);
    if (field == 1 && wire == 2) op->type = r.Bytes();
    else if (field == 2 && wire == 2) op->name = r.Bytes();
    else if (field == 3 && wire == 2) op->input.push_back(r.Bytes());
    else if (field == 4 && wire == 2) op->output.push_back(r.Bytes());
    else if (field == 5 && wire == 2) { op->arg.emplace_back(); if (!ReadArgument(r.Sub(), &op->arg.back())) return false; }
    else if (field == 6 && wire == 2) { op->has_device_option = true; if (!ReadDevice(r.Sub(), &op->device_option)) return false; }
    else r.Skip(wire);
  }
  return r.ok;
}

bool ReadValueInfo(Reader r, ValueInfo* v) {
  while (r.ok && r.p < r.end) {
    uint64_t tag = r.Varint();
    int field = (int)(tag >> 3), wire = (int)(tag & 7);
    if (field == 1 && wire == 2) v->name = r.Bytes();
    else if (field == 2 && wire == 0) v->dtype = (int)r.Varint();
    else if (field == 4 && wire == 0) v->level = (int)r.Varint();
    else if (field == 5 && wire == 0) v->input_type = (int)r.Varint();
    else if (field == 6 && wire == 2) v->feature_name = r.Bytes();
    else r.Skip(wire);
  }
  return r.ok;
}

}  // namespace

bool ParseNetDefBinary(const std::string& bytes, NetDef* out, std::string* err) {
  *out = NetDef();
  Reader r{reinterpret_cast<const uint8_t*>(bytes.data()), reinterpret_cast<const uint8_t*>(bytes.data()) + bytes.size()};
  bool good = true;
  while (good && r.ok && r.p < r.end) {
    uint64_t tag = r.Varint();
    int field = (int)(tag >> 3), wire = (int)(tag & 7);
    if (field == 1 && wire == 2) out->name = r.Bytes();
    else if (field == 2 && wire == 2) { out->op.emplace_back(); good = ReadOperator(r.Sub(), &out->op.back()); }
    else if (field == 3 && wire == 2) out->run_mode = r.Bytes();
    else if (field == 4 && wire == 2) { out->arg.emplace_back(); good = ReadArgument(r.Sub(), &out->arg.back()); }
    else if (field == 5 && wire == 2) good = ReadDevice(r.Sub(), &out->device_option);
    else if (field == 6 && wire == 2) { out->external_input.emplace_back(); good = ReadValueInfo(r.Sub(), &out->external_input.back()); }
    else if (field == 7 && wire == 2) { out->external_output.emplace_back(); good = ReadValueInfo(r.Sub(), &out->external_output.back()); }
    else r.Skip(wire);
  }
  if (!good || !r.ok) { *err = "malformed NetDef protobuf"; return false; }
  return true;
}

const Argument* OperatorDef::FindArg(const std::string& n) const {
  for (const auto& a : arg)
    if (a.name == n) return &a;
  return nullptr;
}

std::string OperatorDef::DebugString() const {
  std::ostringstream os;
  os << " op{type:" << type << " name:" << name << " in:";
  for (const auto& i : input) os << i << ",";
  os << " out:";
  for (const auto& o : output) os << o << ",";
  os << "}";
  return os.str();
}

}  // namespace blaze
