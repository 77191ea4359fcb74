// Minimal JSON reader for graph files.  Malformed text is a runtime error, as with the
// reference's streaming reader (include/utils/json.h), whose checks are CHECK failures.
#pragma once
#include <cctype>
#include <cstdlib>
#include <string>
#include <utility>
#include <vector>
#include "base.h"

namespace cvm {

struct JValue {
  enum Type { kNull, kBool, kNumber, kString, kArray, kObject } type = kNull;
  bool b = false;
  std::string s;  // string payload, or the literal text of a number
  std::vector<JValue> arr;
  std::vector<std::pair<std::string, JValue>> obj;

  bool is_string() const { return type == kString; }
  bool is_array() const { return type == kArray; }
  bool is_object() const { return type == kObject; }
  const std::string& as_string() const {
    CHECK(type == kString) << "invalid json format: expected a string";
    return s;
  }
  int64_t as_int() const {
    CHECK(type == kNumber) << "invalid json format: expected a number";
    char* end = nullptr;
    long long v = strtoll(s.c_str(), &end, 10);
    CHECK(end && *end == 0) << "invalid json format: expected an integer, got " << s;
    return v;
  }
  const std::vector<JValue>& as_array() const {
    CHECK(type == kArray) << "invalid json format: expected an array";
    return arr;
  }
};

class JsonParser {
 public:
  explicit JsonParser(const std::string& text) : t_(text), p_(0) {}
  JValue parse() {
    JValue v = value();
    return v;
  }

 private:
  const std::string& t_;
  size_t p_;
  void ws() {
    while (p_ < t_.size() && isspace((unsigned char)t_[p_])) ++p_;
  }
  char peek() {
    ws();
    CHECK(p_ < t_.size()) << "invalid json format: unexpected end of text";
    return t_[p_];
  }
  void expect(char c) {
    char g = peek();
    CHECK(g == c) << "invalid json format: expected '" << c << "' at offset " << p_ << ", got '" << g << "'";
    ++p_;
  }
  JValue value() {
    char c = peek();
    JValue v;
    if (c == '{') {
      v.type = JValue::kObject;
      ++p_;
      if (peek() == '}') { ++p_; return v; }
      while (true) {
        JValue k = string_value();
        expect(':');
        JValue val = value();
        v.obj.emplace_back(k.s, std::move(val));
        char d = peek();
        if (d == ',') { ++p_; continue; }
        expect('}');
        break;
      }
    } else if (c == '[') {
      v.type = JValue::kArray;
      ++p_;
      if (peek() == ']') { ++p_; return v; }
      while (true) {
        v.arr.push_back(value());
        char d = peek();
        if (d == ',') { ++p_; continue; }
        expect(']');
        break;
      }
    } else if (c == '"') {
      v = string_value();
    } else if (c == 't' && t_.compare(p_, 4, "true") == 0) {
      v.type = JValue::kBool; v.b = true; p_ += 4;
    } else if (c == 'f' && t_.compare(p_, 5, "false") == 0) {
      v.type = JValue::kBool; v.b = false; p_ += 5;
    } else if (c == 'n' && t_.compare(p_, 4, "null") == 0) {
      v.type = JValue::kNull; p_ += 4;
    } else {
      size_t b = p_;
      if (t_[p_] == '-' || t_[p_] == '+') ++p_;
      while (p_ < t_.size() && (isdigit((unsigned char)t_[p_]) || t_[p_] == '.' || t_[p_] == 'e' ||
                                t_[p_] == 'E' || t_[p_] == '-' || t_[p_] == '+'))
        ++p_;
      CHECK(p_ > b) << "invalid json format: unexpected character '" << c << "' at offset " << b;
      v.type = JValue::kNumber;
      v.s = t_.substr(b, p_ - b);
    }
    return v;
  }
  JValue string_value() {
    expect('"');
    JValue v;
    v.type = JValue::kString;
    while (true) {
      CHECK(p_ < t_.size()) << "invalid json format: unterminated string";
      char c = t_[p_++];
      if (c == '"') break;
      if (c == '\\') {
        CHECK(p_ < t_.size()) << "invalid json format: unterminated escape";
        char e = t_[p_++];
        switch (e) {
          case 'n': v.s.push_back('\n'); break;
          case 't': v.s.push_back('\t'); break;
          case 'r': v.s.push_back('\r'); break;
          case 'b': v.s.push_back('\b'); break;
          case 'f': v.s.push_back('\f'); break;
          case '\\': v.s.push_back('\\'); break;
          case '/': v.s.push_back('/'); break;
          case '"': v.s.push_back('"'); break;
          case 'u': {
            CHECK(p_ + 4 <= t_.size()) << "invalid json format: bad \\u escape";
            unsigned code = (unsigned)strtoul(t_.substr(p_, 4).c_str(), nullptr, 16);
            p_ += 4;
            if (code < 0x80) v.s.push_back((char)code);
            else if (code < 0x800) { v.s.push_back((char)(0xC0 | (code >> 6))); v.s.push_back((char)(0x80 | (code & 0x3F))); }
            else { v.s.push_back((char)(0xE0 | (code >> 12))); v.s.push_back((char)(0x80 | ((code >> 6) & 0x3F))); v.s.push_back((char)(0x80 | (code & 0x3F))); }
          } break;
          default: FATAL() << "invalid json format: unknown escape \\" << e;
        }
      } else {
        v.s.push_back(c);
      }
    }
    return v;
  }
};

inline JValue parse_json(const std::string& text) { return JsonParser(text).parse(); }

}  // namespace cvm
