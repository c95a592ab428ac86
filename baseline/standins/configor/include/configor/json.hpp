// Stand-in for the slice of configor 0.9 that the reference's checkpoint writer uses
// (kraken/checkpoint/checkpoint.cc:288-403): a JSON value that can be built with operator[],
// assignment from numbers / strings / string maps / integer vectors, array({}) + push_back, and
// dump(indent, indent_char).  Object keys keep insertion order.  Header only.
#pragma once

#include <cstdint>
#include <initializer_list>
#include <sstream>
#include <string>
#include <type_traits>
#include <unordered_map>
#include <map>
#include <utility>
#include <vector>

namespace configor {

class json {
public:
  enum class Kind { kNull, kBool, kInt, kUint, kFloat, kString, kArray, kObject };

  json() : kind_(Kind::kNull) {}
  json(bool v) : kind_(Kind::kBool), b_(v) {}
  template <typename I, typename std::enable_if<std::is_integral<I>::value && std::is_signed<I>::value, int>::type = 0>
  json(I v) : kind_(Kind::kInt), i_(static_cast<int64_t>(v)) {}
  template <typename U, typename std::enable_if<std::is_integral<U>::value && std::is_unsigned<U>::value &&
                                                !std::is_same<U, bool>::value, long>::type = 0>
  json(U v) : kind_(Kind::kUint), u_(static_cast<uint64_t>(v)) {}
  json(double v) : kind_(Kind::kFloat), f_(v) {}
  json(float v) : kind_(Kind::kFloat), f_(v) {}
  json(const char* s) : kind_(Kind::kString), s_(s) {}
  json(const std::string& s) : kind_(Kind::kString), s_(s) {}
  template <typename V>
  json(const std::vector<V>& v) : kind_(Kind::kArray) {
    for (const auto& x : v) items_.emplace_back(json(x));
  }
  template <typename V>
  json(const std::unordered_map<std::string, V>& m) : kind_(Kind::kObject) {
    for (const auto& kv : m) (*this)[kv.first] = json(kv.second);
  }
  template <typename V>
  json(const std::map<std::string, V>& m) : kind_(Kind::kObject) {
    for (const auto& kv : m) (*this)[kv.first] = json(kv.second);
  }

  static json array(std::initializer_list<json> init) {
    json j;
    j.kind_ = Kind::kArray;
    j.items_.assign(init.begin(), init.end());
    return j;
  }
  static json object() {
    json j;
    j.kind_ = Kind::kObject;
    return j;
  }

  json& operator[](const std::string& key) {
    if (kind_ == Kind::kNull) kind_ = Kind::kObject;
    for (auto& kv : members_)
      if (kv.first == key) return kv.second;
    members_.emplace_back(key, json());
    return members_.back().second;
  }
  json& operator[](const char* key) { return (*this)[std::string(key)]; }

  void push_back(json v) {
    if (kind_ == Kind::kNull) kind_ = Kind::kArray;
    items_.emplace_back(std::move(v));
  }

  size_t size() const { return kind_ == Kind::kArray ? items_.size() : members_.size(); }

  std::string dump(int indent = -1, char indent_char = ' ') const {
    std::ostringstream os;
    write(os, indent, indent_char, 0);
    return os.str();
  }

private:
  static void escape(std::ostream& os, const std::string& s) {
    os << '"';
    for (unsigned char c : s) {
      switch (c) {
        case '"': os << "\\\""; break;
        case '\\': os << "\\\\"; break;
        case '\n': os << "\\n"; break;
        case '\r': os << "\\r"; break;
        case '\t': os << "\\t"; break;
        default:
          if (c < 0x20) {
            static const char* hex = "0123456789abcdef";
            os << "\\u00" << hex[c >> 4] << hex[c & 15];
          } else {
            os << static_cast<char>(c);
          }
      }
    }
    os << '"';
  }
  static void pad(std::ostream& os, int indent, char ch, int depth) {
    if (indent < 0) return;
    os << '\n';
    for (int i = 0; i < indent * depth; ++i) os << ch;
  }
  void write(std::ostream& os, int indent, char ch, int depth) const {
    switch (kind_) {
      case Kind::kNull: os << "null"; break;
      case Kind::kBool: os << (b_ ? "true" : "false"); break;
      case Kind::kInt: os << i_; break;
      case Kind::kUint: os << u_; break;
      case Kind::kFloat: os << f_; break;
      case Kind::kString: escape(os, s_); break;
      case Kind::kArray:
        if (items_.empty()) { os << "[]"; break; }
        os << '[';
        for (size_t i = 0; i < items_.size(); ++i) {
          if (i) os << ',';
          pad(os, indent, ch, depth + 1);
          items_[i].write(os, indent, ch, depth + 1);
        }
        pad(os, indent, ch, depth);
        os << ']';
        break;
      case Kind::kObject:
        if (members_.empty()) { os << "{}"; break; }
        os << '{';
        for (size_t i = 0; i < members_.size(); ++i) {
          if (i) os << ',';
          pad(os, indent, ch, depth + 1);
          escape(os, members_[i].first);
          os << (indent < 0 ? ":" : ": ");
          members_[i].second.write(os, indent, ch, depth + 1);
        }
        pad(os, indent, ch, depth);
        os << '}';
        break;
    }
  }

  Kind kind_;
  bool b_ = false;
  int64_t i_ = 0;
  uint64_t u_ = 0;
  double f_ = 0.0;
  std::string s_;
  std::vector<json> items_;
  std::vector<std::pair<std::string, json>> members_;
};

}  // namespace configor
