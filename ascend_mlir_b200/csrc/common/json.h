// Minimal self-contained JSON value, parser and writer (C++17, no dependencies).
// Used for launch descriptors, tiling_space.json, run manifests and profile traces.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace afir {
namespace json {

class Value;
using Array = std::vector<Value>;
// Objects keep insertion order: tiling field order is part of the kernel ABI.
using Member = std::pair<std::string, Value>;
using Object = std::vector<Member>;

class Value {
public:
  enum class Kind { Null, Bool, Int, Double, String, Array, Object };

  Value() = default;
  Value(std::nullptr_t) {}
  Value(bool b) : kind_(Kind::Bool), b_(b) {}
  Value(int v) : kind_(Kind::Int), i_(v) {}
  Value(int64_t v) : kind_(Kind::Int), i_(v) {}
  Value(uint64_t v) : kind_(Kind::Int), i_(static_cast<int64_t>(v)) {}
  Value(double v) : kind_(Kind::Double), d_(v) {}
  Value(const char *s) : kind_(Kind::String), s_(s) {}
  Value(std::string s) : kind_(Kind::String), s_(std::move(s)) {}
  Value(Array a) : kind_(Kind::Array), a_(std::make_shared<Array>(std::move(a))) {}
  Value(Object o) : kind_(Kind::Object), o_(std::make_shared<Object>(std::move(o))) {}

  Kind kind() const { return kind_; }
  bool isNull() const { return kind_ == Kind::Null; }
  bool isBool() const { return kind_ == Kind::Bool; }
  bool isInt() const { return kind_ == Kind::Int; }
  bool isNumber() const { return kind_ == Kind::Int || kind_ == Kind::Double; }
  bool isString() const { return kind_ == Kind::String; }
  bool isArray() const { return kind_ == Kind::Array; }
  bool isObject() const { return kind_ == Kind::Object; }

  bool asBool() const { return b_; }
  int64_t asInt() const { return kind_ == Kind::Double ? static_cast<int64_t>(d_) : i_; }
  double asDouble() const { return kind_ == Kind::Int ? static_cast<double>(i_) : d_; }
  const std::string &asString() const { return s_; }
  const Array &asArray() const { return *a_; }
  Array &asArray() { return *a_; }
  const Object &asObject() const { return *o_; }
  Object &asObject() { return *o_; }

  // Object lookup; returns nullptr when absent or when this is not an object.
  const Value *find(const std::string &key) const {
    if (kind_ != Kind::Object) return nullptr;
    for (const auto &m : *o_)
      if (m.first == key) return &m.second;
    return nullptr;
  }
  void set(const std::string &key, Value v) {
    if (kind_ != Kind::Object) { kind_ = Kind::Object; o_ = std::make_shared<Object>(); }
    for (auto &m : *o_)
      if (m.first == key) { m.second = std::move(v); return; }
    o_->emplace_back(key, std::move(v));
  }
  void push(Value v) {
    if (kind_ != Kind::Array) { kind_ = Kind::Array; a_ = std::make_shared<Array>(); }
    a_->push_back(std::move(v));
  }

  std::string getString(const std::string &key, const std::string &dflt = "") const {
    const Value *v = find(key);
    return v && v->isString() ? v->asString() : dflt;
  }
  int64_t getInt(const std::string &key, int64_t dflt = 0) const {
    const Value *v = find(key);
    return v && v->isNumber() ? v->asInt() : dflt;
  }
  double getDouble(const std::string &key, double dflt = 0.0) const {
    const Value *v = find(key);
    return v && v->isNumber() ? v->asDouble() : dflt;
  }
  bool getBool(const std::string &key, bool dflt = false) const {
    const Value *v = find(key);
    return v && v->isBool() ? v->asBool() : dflt;
  }

private:
  Kind kind_ = Kind::Null;
  bool b_ = false;
  int64_t i_ = 0;
  double d_ = 0.0;
  std::string s_;
  std::shared_ptr<Array> a_;
  std::shared_ptr<Object> o_;
};

// Parses `text`; on failure returns false and describes the problem (with byte offset) in `error`.
bool parse(const std::string &text, Value &out, std::string &error);

// Serialises `v`. indent < 0: compact one-line form; otherwise pretty-printed.
std::string dump(const Value &v, int indent = -1);

} // namespace json
} // namespace afir
