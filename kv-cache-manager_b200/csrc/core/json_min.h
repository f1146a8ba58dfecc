// A small JSON reader: enough for the header of a safetensors file (objects, arrays, strings with
// escapes, numbers, true / false / null).  Values keep the order of their keys.  Errors throw
// std::runtime_error with the byte offset.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace kvcm {
namespace json {

struct Value {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool boolean = false;
  double number = 0.0;
  bool is_integer = false;
  long long integer = 0;
  std::string text;
  std::vector<Value> items;
  std::vector<std::pair<std::string, Value>> members;

  const Value* find(const std::string& key) const {
    for (const auto& m : members)
      if (m.first == key) return &m.second;
    return nullptr;
  }
};

class Parser {
 public:
  Parser(const char* data, size_t size) : p_(data), end_(data + size), begin_(data) {}

  Value parse_document() {
    Value v = parse_value(0);
    skip_space();
    if (p_ != end_) fail("text after the value");
    return v;
  }

 private:
  const char* p_;
  const char* end_;
  const char* begin_;

  [[noreturn]] void fail(const char* what) const {
    throw std::runtime_error(std::string(what) + " at byte " + std::to_string(p_ - begin_));
  }
  void skip_space() {
    while (p_ != end_ && (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r')) ++p_;
  }
  bool take(char c) {
    skip_space();
    if (p_ != end_ && *p_ == c) { ++p_; return true; }
    return false;
  }
  void expect_word(const char* w) {
    for (const char* q = w; *q; ++q, ++p_)
      if (p_ == end_ || *p_ != *q) fail("unknown literal");
  }
  static void append_utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out += char(cp);
    else if (cp < 0x800) { out += char(0xC0 | (cp >> 6)); out += char(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { out += char(0xE0 | (cp >> 12)); out += char(0x80 | ((cp >> 6) & 0x3F)); out += char(0x80 | (cp & 0x3F)); }
    else { out += char(0xF0 | (cp >> 18)); out += char(0x80 | ((cp >> 12) & 0x3F)); out += char(0x80 | ((cp >> 6) & 0x3F)); out += char(0x80 | (cp & 0x3F)); }
  }
  uint32_t hex4() {
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i, ++p_) {
      if (p_ == end_) fail("short \\u escape");
      const char c = *p_;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= uint32_t(c - '0');
      else if (c >= 'a' && c <= 'f') v |= uint32_t(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') v |= uint32_t(c - 'A' + 10);
      else fail("bad \\u escape");
    }
    return v;
  }
  std::string parse_string() {
    if (!take('"')) fail("expected a string");
    std::string out;
    while (true) {
      if (p_ == end_) fail("unterminated string");
      const char c = *p_++;
      if (c == '"') return out;
      if (static_cast<unsigned char>(c) < 0x20) fail("control character in a string");
      if (c != '\\') { out += c; continue; }
      if (p_ == end_) fail("unterminated escape");
      const char e = *p_++;
      switch (e) {
        case '"': out += '"'; break;
        case '\\': out += '\\'; break;
        case '/': out += '/'; break;
        case 'b': out += '\b'; break;
        case 'f': out += '\f'; break;
        case 'n': out += '\n'; break;
        case 'r': out += '\r'; break;
        case 't': out += '\t'; break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
            p_ += 2;
            const uint32_t lo = hex4();
            if (lo >= 0xDC00 && lo < 0xE000) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            else fail("bad surrogate pair");
          }
          append_utf8(out, cp);
          break;
        }
        default: fail("unknown escape");
      }
    }
  }
  Value parse_number() {
    const char* start = p_;
    bool integer = true;
    if (p_ != end_ && *p_ == '-') ++p_;
    if (p_ == end_ || *p_ < '0' || *p_ > '9') fail("bad number");
    while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
    if (p_ != end_ && *p_ == '.') {
      integer = false;
      ++p_;
      if (p_ == end_ || *p_ < '0' || *p_ > '9') fail("bad number");
      while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
    }
    if (p_ != end_ && (*p_ == 'e' || *p_ == 'E')) {
      integer = false;
      ++p_;
      if (p_ != end_ && (*p_ == '+' || *p_ == '-')) ++p_;
      if (p_ == end_ || *p_ < '0' || *p_ > '9') fail("bad number");
      while (p_ != end_ && *p_ >= '0' && *p_ <= '9') ++p_;
    }
    const std::string text(start, p_);
    Value v;
    v.kind = Value::Number;
    v.number = std::strtod(text.c_str(), nullptr);
    if (integer && text.size() <= 18) {
      v.is_integer = true;
      v.integer = std::strtoll(text.c_str(), nullptr, 10);
    }
    return v;
  }
  Value parse_value(int depth) {
    if (depth > 64) fail("nested too deeply");
    skip_space();
    if (p_ == end_) fail("unexpected end");
    Value v;
    const char c = *p_;
    if (c == '{') {
      ++p_;
      v.kind = Value::Object;
      if (take('}')) return v;
      do {
        skip_space();
        std::string key = parse_string();
        if (!take(':')) fail("expected ':'");
        v.members.emplace_back(std::move(key), parse_value(depth + 1));
      } while (take(','));
      if (!take('}')) fail("expected '}'");
    } else if (c == '[') {
      ++p_;
      v.kind = Value::Array;
      if (take(']')) return v;
      do v.items.push_back(parse_value(depth + 1));
      while (take(','));
      if (!take(']')) fail("expected ']'");
    } else if (c == '"') {
      v.kind = Value::String;
      v.text = parse_string();
    } else if (c == 't') { expect_word("true"); v.kind = Value::Bool; v.boolean = true; }
    else if (c == 'f') { expect_word("false"); v.kind = Value::Bool; }
    else if (c == 'n') { expect_word("null"); }
    else v = parse_number();
    return v;
  }
};

}  // namespace json
}  // namespace kvcm
