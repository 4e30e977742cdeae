// Minimal JSON document model (parse + dump).  The control plane, endpoint documents and schedule
// files are JSON (the reference used nlohmann::json for the same purposes, csrc/cluster/daemon.cc:4;
// that submodule is an empty directory and there is no network, so this is self-contained).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace pccl {

class Json {
 public:
  enum class Kind { Null, Bool, Number, String, Array, Object };
  using Array = std::vector<Json>;
  using Object = std::vector<std::pair<std::string, Json>>;   // keeps insertion order

  Json() : kind_(Kind::Null) {}
  Json(std::nullptr_t) : kind_(Kind::Null) {}
  Json(bool b) : kind_(Kind::Bool), b_(b) {}
  Json(int v) : kind_(Kind::Number), n_(v), is_int_(true), i_(v) {}
  Json(int64_t v) : kind_(Kind::Number), n_(static_cast<double>(v)), is_int_(true), i_(v) {}
  Json(uint64_t v) : kind_(Kind::Number), n_(static_cast<double>(v)), is_int_(true), i_(static_cast<int64_t>(v)) {}
  Json(double v) : kind_(Kind::Number), n_(v) {}
  Json(const char* s) : kind_(Kind::String), s_(s) {}
  Json(const std::string& s) : kind_(Kind::String), s_(s) {}
  static Json array() { Json j; j.kind_ = Kind::Array; return j; }
  static Json object() { Json j; j.kind_ = Kind::Object; return j; }

  Kind kind() const { return kind_; }
  bool isNull() const { return kind_ == Kind::Null; }
  bool isObject() const { return kind_ == Kind::Object; }
  bool isArray() const { return kind_ == Kind::Array; }
  bool isString() const { return kind_ == Kind::String; }
  bool isNumber() const { return kind_ == Kind::Number; }

  bool asBool(bool d = false) const { return kind_ == Kind::Bool ? b_ : (kind_ == Kind::Number ? n_ != 0 : d); }
  int64_t asInt(int64_t d = 0) const { return kind_ == Kind::Number ? (is_int_ ? i_ : static_cast<int64_t>(n_)) : d; }
  double asDouble(double d = 0) const { return kind_ == Kind::Number ? n_ : d; }
  const std::string& asString() const { static const std::string e; return kind_ == Kind::String ? s_ : e; }

  // arrays
  size_t size() const { return kind_ == Kind::Array ? a_.size() : (kind_ == Kind::Object ? o_.size() : 0); }
  const Json& at(size_t i) const { return a_.at(i); }
  Json& push(Json v) { a_.push_back(std::move(v)); return a_.back(); }
  const Array& items() const { return a_; }

  // objects
  bool contains(const std::string& k) const { return find(k) != nullptr; }
  const Json* find(const std::string& k) const {
    for (auto& kv : o_) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  const Json& operator[](const std::string& k) const {
    static const Json null_json;
    const Json* p = find(k);
    return p ? *p : null_json;
  }
  Json& set(const std::string& k, Json v) {
    for (auto& kv : o_) if (kv.first == k) { kv.second = std::move(v); return kv.second; }
    o_.emplace_back(k, std::move(v));
    return o_.back().second;
  }
  const Object& members() const { return o_; }

  std::string dump() const;
  static Json parse(const std::string& text);   // throws std::runtime_error
  static Json parseFile(const std::string& path);

 private:
  Kind kind_;
  bool b_ = false;
  double n_ = 0;
  bool is_int_ = false;
  int64_t i_ = 0;
  std::string s_;
  Array a_;
  Object o_;
  void dumpTo(std::string& out) const;
};

}  // namespace pccl
