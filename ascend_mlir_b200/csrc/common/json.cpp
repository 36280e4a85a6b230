#include "common/json.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace afir {
namespace json {
namespace {

class Parser {
public:
  Parser(const std::string &text, std::string &error) : s_(text), err_(error) {}

  bool run(Value &out) {
    skipWs();
    if (!value(out, 0)) return false;
    skipWs();
    if (pos_ != s_.size()) return fail("trailing characters after JSON value");
    return true;
  }

private:
  const std::string &s_;
  std::string &err_;
  size_t pos_ = 0;

  bool fail(const char *msg) {
    err_ = std::string(msg) + " at offset " + std::to_string(pos_);
    return false;
  }
  void skipWs() {
    while (pos_ < s_.size()) {
      char c = s_[pos_];
      if (c == ' ' || c == '\t' || c == '\n' || c == '\r') ++pos_;
      else break;
    }
  }
  bool literal(const char *word) {
    size_t n = std::strlen(word);
    if (s_.compare(pos_, n, word) != 0) return fail("invalid literal");
    pos_ += n;
    return true;
  }
  static void appendUtf8(std::string &out, uint32_t cp) {
    if (cp < 0x80) out.push_back(static_cast<char>(cp));
    else if (cp < 0x800) {
      out.push_back(static_cast<char>(0xC0 | (cp >> 6)));
      out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
      out.push_back(static_cast<char>(0xE0 | (cp >> 12)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    } else {
      out.push_back(static_cast<char>(0xF0 | (cp >> 18)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 12) & 0x3F)));
      out.push_back(static_cast<char>(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back(static_cast<char>(0x80 | (cp & 0x3F)));
    }
  }
  bool hex4(uint32_t &cp) {
    if (pos_ + 4 > s_.size()) return fail("truncated \\u escape");
    cp = 0;
    for (int i = 0; i < 4; ++i) {
      char c = s_[pos_++];
      cp <<= 4;
      if (c >= '0' && c <= '9') cp |= static_cast<uint32_t>(c - '0');
      else if (c >= 'a' && c <= 'f') cp |= static_cast<uint32_t>(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') cp |= static_cast<uint32_t>(c - 'A' + 10);
      else return fail("bad hex digit in \\u escape");
    }
    return true;
  }
  bool string(std::string &out) {
    ++pos_; // opening quote
    while (true) {
      if (pos_ >= s_.size()) return fail("unterminated string");
      char c = s_[pos_++];
      if (c == '"') return true;
      if (c != '\\') { out.push_back(c); continue; }
      if (pos_ >= s_.size()) return fail("unterminated escape");
      char e = s_[pos_++];
      switch (e) {
      case '"': out.push_back('"'); break;
      case '\\': out.push_back('\\'); break;
      case '/': out.push_back('/'); break;
      case 'b': out.push_back('\b'); break;
      case 'f': out.push_back('\f'); break;
      case 'n': out.push_back('\n'); break;
      case 'r': out.push_back('\r'); break;
      case 't': out.push_back('\t'); break;
      case 'u': {
        uint32_t cp;
        if (!hex4(cp)) return false;
        if (cp >= 0xD800 && cp <= 0xDBFF && s_.compare(pos_, 2, "\\u") == 0) {
          pos_ += 2;
          uint32_t lo;
          if (!hex4(lo)) return false;
          cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
        }
        appendUtf8(out, cp);
        break;
      }
      default: return fail("unknown escape");
      }
    }
  }
  bool number(Value &out) {
    size_t start = pos_;
    bool isDouble = false;
    if (s_[pos_] == '-') ++pos_;
    while (pos_ < s_.size()) {
      char c = s_[pos_];
      if (c >= '0' && c <= '9') ++pos_;
      else if (c == '.' || c == 'e' || c == 'E' || c == '+' || c == '-') { isDouble = true; ++pos_; }
      else break;
    }
    std::string tok = s_.substr(start, pos_ - start);
    if (tok.empty() || tok == "-") return fail("invalid number");
    char *end = nullptr;
    if (!isDouble) {
      errno = 0;
      long long v = std::strtoll(tok.c_str(), &end, 10);
      if (end && *end == '\0' && errno == 0) { out = Value(static_cast<int64_t>(v)); return true; }
    }
    double d = std::strtod(tok.c_str(), &end);
    if (!end || *end != '\0') return fail("invalid number");
    out = Value(d);
    return true;
  }
  bool value(Value &out, int depth) {
    if (depth > 64) return fail("nesting too deep");
    if (pos_ >= s_.size()) return fail("unexpected end of input");
    char c = s_[pos_];
    if (c == '{') {
      ++pos_;
      Object obj;
      skipWs();
      if (pos_ < s_.size() && s_[pos_] == '}') { ++pos_; out = Value(std::move(obj)); return true; }
      while (true) {
        skipWs();
        if (pos_ >= s_.size() || s_[pos_] != '"') return fail("expected object key");
        std::string key;
        if (!string(key)) return false;
        skipWs();
        if (pos_ >= s_.size() || s_[pos_] != ':') return fail("expected ':'");
        ++pos_;
        skipWs();
        Value v;
        if (!value(v, depth + 1)) return false;
        obj.emplace_back(std::move(key), std::move(v));
        skipWs();
        if (pos_ < s_.size() && s_[pos_] == ',') { ++pos_; continue; }
        if (pos_ < s_.size() && s_[pos_] == '}') { ++pos_; break; }
        return fail("expected ',' or '}'");
      }
      out = Value(std::move(obj));
      return true;
    }
    if (c == '[') {
      ++pos_;
      Array arr;
      skipWs();
      if (pos_ < s_.size() && s_[pos_] == ']') { ++pos_; out = Value(std::move(arr)); return true; }
      while (true) {
        skipWs();
        Value v;
        if (!value(v, depth + 1)) return false;
        arr.push_back(std::move(v));
        skipWs();
        if (pos_ < s_.size() && s_[pos_] == ',') { ++pos_; continue; }
        if (pos_ < s_.size() && s_[pos_] == ']') { ++pos_; break; }
        return fail("expected ',' or ']'");
      }
      out = Value(std::move(arr));
      return true;
    }
    if (c == '"') {
      std::string str;
      if (!string(str)) return false;
      out = Value(std::move(str));
      return true;
    }
    if (c == 't') { if (!literal("true")) return false; out = Value(true); return true; }
    if (c == 'f') { if (!literal("false")) return false; out = Value(false); return true; }
    if (c == 'n') { if (!literal("null")) return false; out = Value(nullptr); return true; }
    if (c == '-' || (c >= '0' && c <= '9')) return number(out);
    return fail("unexpected character");
  }
};

void dumpString(const std::string &s, std::string &out) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
    case '"': out += "\\\""; break;
    case '\\': out += "\\\\"; break;
    case '\n': out += "\\n"; break;
    case '\r': out += "\\r"; break;
    case '\t': out += "\\t"; break;
    default:
      if (c < 0x20) {
        char buf[8];
        std::snprintf(buf, sizeof(buf), "\\u%04x", c);
        out += buf;
      } else out.push_back(static_cast<char>(c));
    }
  }
  out.push_back('"');
}

void dumpValue(const Value &v, int indent, int level, std::string &out) {
  auto newline = [&](int lvl) {
    if (indent < 0) return;
    out.push_back('\n');
    out.append(static_cast<size_t>(indent * lvl), ' ');
  };
  switch (v.kind()) {
  case Value::Kind::Null: out += "null"; break;
  case Value::Kind::Bool: out += v.asBool() ? "true" : "false"; break;
  case Value::Kind::Int: out += std::to_string(v.asInt()); break;
  case Value::Kind::Double: {
    double d = v.asDouble();
    if (!std::isfinite(d)) { out += "null"; break; }
    char buf[40];
    std::snprintf(buf, sizeof(buf), "%.17g", d);
    // keep doubles recognisable as doubles
    if (!std::strpbrk(buf, ".eE")) std::strcat(buf, ".0");
    out += buf;
    break;
  }
  case Value::Kind::String: dumpString(v.asString(), out); break;
  case Value::Kind::Array: {
    const Array &a = v.asArray();
    if (a.empty()) { out += "[]"; break; }
    out.push_back('[');
    for (size_t i = 0; i < a.size(); ++i) {
      if (i) out += indent < 0 ? "," : ",";
      newline(level + 1);
      dumpValue(a[i], indent, level + 1, out);
    }
    newline(level);
    out.push_back(']');
    break;
  }
  case Value::Kind::Object: {
    const Object &o = v.asObject();
    if (o.empty()) { out += "{}"; break; }
    out.push_back('{');
    for (size_t i = 0; i < o.size(); ++i) {
      if (i) out.push_back(',');
      newline(level + 1);
      dumpString(o[i].first, out);
      out += indent < 0 ? ":" : ": ";
      dumpValue(o[i].second, indent, level + 1, out);
    }
    newline(level);
    out.push_back('}');
    break;
  }
  }
}

} // namespace

bool parse(const std::string &text, Value &out, std::string &error) {
  Parser p(text, error);
  return p.run(out);
}

std::string dump(const Value &v, int indent) {
  std::string out;
  dumpValue(v, indent, 0, out);
  return out;
}

} // namespace json
} // namespace afir
