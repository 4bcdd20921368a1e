// A small JSON reader (RFC 8259 subset sufficient for model files): objects, arrays,
// strings with escapes, numbers (kept as double), true/false/null.  The reference
// uses a vendored third-party JSON library for the same job (src/json/xgboostparser.h:56-60).
#pragma once
#include <cstdint>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace tb {
namespace json {

struct Value;
using Array = std::vector<Value>;
using Object = std::map<std::string, Value>;

struct Value {
  enum Kind { kNull, kBool, kNumber, kString, kArray, kObject } kind = kNull;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::shared_ptr<Array> arr;
  std::shared_ptr<Object> obj;

  bool is_object() const { return kind == kObject; }
  bool is_array() const { return kind == kArray; }
  bool has(const std::string &k) const { return kind == kObject && obj->count(k); }
  const Value &at(const std::string &k) const {
    if (kind != kObject) throw std::runtime_error("JSON: not an object while reading \"" + k + "\"");
    auto it = obj->find(k);
    if (it == obj->end()) throw std::runtime_error("JSON: missing key \"" + k + "\"");
    return it->second;
  }
  const Array &array() const {
    if (kind != kArray) throw std::runtime_error("JSON: not an array");
    return *arr;
  }
  // numbers may be stored as JSON numbers or as strings (XGBoost writes parameters
  // as strings)
  double number() const {
    if (kind == kNumber) return num;
    if (kind == kBool) return b ? 1.0 : 0.0;
    if (kind == kString) return std::strtod(str.c_str(), nullptr);
    throw std::runtime_error("JSON: not a number");
  }
  const std::string &string() const {
    if (kind != kString) throw std::runtime_error("JSON: not a string");
    return str;
  }
};

class Parser {
public:
  Parser(const char *begin, const char *end) : p_(begin), end_(end) {}
  Value parse() {
    Value v = value();
    ws();
    if (p_ != end_) error("trailing characters");
    return v;
  }

private:
  const char *p_, *end_;
  [[noreturn]] void error(const std::string &what) const { throw std::runtime_error("JSON: " + what); }
  void ws() {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
  }
  bool eat(char c) {
    ws();
    if (p_ < end_ && *p_ == c) { ++p_; return true; }
    return false;
  }
  Value value() {
    ws();
    if (p_ >= end_) error("unexpected end of input");
    Value v;
    switch (*p_) {
    case '{': {
      ++p_;
      v.kind = Value::kObject;
      v.obj = std::make_shared<Object>();
      if (eat('}')) return v;
      do {
        ws();
        if (p_ >= end_ || *p_ != '"') error("expected a key");
        std::string k = string();
        if (!eat(':')) error("expected ':'");
        (*v.obj)[k] = value();
      } while (eat(','));
      if (!eat('}')) error("expected '}'");
      return v;
    }
    case '[': {
      ++p_;
      v.kind = Value::kArray;
      v.arr = std::make_shared<Array>();
      if (eat(']')) return v;
      do { v.arr->push_back(value()); } while (eat(','));
      if (!eat(']')) error("expected ']'");
      return v;
    }
    case '"':
      v.kind = Value::kString;
      v.str = string();
      return v;
    case 't':
      literal("true");
      v.kind = Value::kBool;
      v.b = true;
      return v;
    case 'f':
      literal("false");
      v.kind = Value::kBool;
      return v;
    case 'n':
      literal("null");
      return v;
    default: {
      char *stop = nullptr;
      v.num = std::strtod(p_, &stop);
      if (stop == p_) error("unexpected character");
      p_ = stop;
      v.kind = Value::kNumber;
      return v;
    }
    }
  }
  void literal(const char *word) {
    for (const char *w = word; *w; ++w, ++p_)
      if (p_ >= end_ || *p_ != *w) error("bad literal");
  }
  std::string string() {
    ++p_; // opening quote
    std::string s;
    while (p_ < end_ && *p_ != '"') {
      if (*p_ == '\\') {
        if (++p_ >= end_) break;
        switch (*p_) {
        case 'n': s += '\n'; break;
        case 't': s += '\t'; break;
        case 'r': s += '\r'; break;
        case 'b': s += '\b'; break;
        case 'f': s += '\f'; break;
        case 'u': {
          if (end_ - p_ < 5) error("bad \\u escape");
          unsigned cp = (unsigned)std::strtoul(std::string(p_ + 1, p_ + 5).c_str(), nullptr, 16);
          p_ += 4;
          if (cp < 0x80) s += (char)cp;
          else if (cp < 0x800) { s += (char)(0xC0 | (cp >> 6)); s += (char)(0x80 | (cp & 0x3F)); }
          else { s += (char)(0xE0 | (cp >> 12)); s += (char)(0x80 | ((cp >> 6) & 0x3F)); s += (char)(0x80 | (cp & 0x3F)); }
          break;
        }
        default: s += *p_;
        }
        ++p_;
      } else {
        s += *p_++;
      }
    }
    if (p_ >= end_) error("unterminated string");
    ++p_; // closing quote
    return s;
  }
};

inline Value parse(const std::string &text) { return Parser(text.data(), text.data() + text.size()).parse(); }

} // namespace json
} // namespace tb
