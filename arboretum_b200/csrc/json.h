// Minimal JSON value, parser and writer (objects keep keys sorted, numbers are
// doubles written in their shortest round-trip form, non-finite numbers are
// written as null) -- enough for the configuration and model documents of the
// reference (src/core/json_conversion.h, src/core/model_helper.cpp), which uses
// nlohmann::json with the same conventions.
#pragma once
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace arb {

struct Json {
  enum Type { Null, Bool, Num, Str, Arr, Obj } type = Null;
  bool b = false;
  double num = 0;
  bool is_int = false;
  std::string str;
  std::vector<Json> arr;
  std::map<std::string, Json> obj;

  Json() {}
  static Json boolean(bool v) {
    Json j;
    j.type = Bool;
    j.b = v;
    return j;
  }
  static Json number(double v) {
    Json j;
    j.type = Num;
    j.num = v;
    return j;
  }
  static Json integer(long long v) {
    Json j;
    j.type = Num;
    j.num = double(v);
    j.is_int = true;
    return j;
  }
  static Json string(const std::string &s) {
    Json j;
    j.type = Str;
    j.str = s;
    return j;
  }
  static Json array() {
    Json j;
    j.type = Arr;
    return j;
  }
  static Json object() {
    Json j;
    j.type = Obj;
    return j;
  }
  bool has(const std::string &k) const { return type == Obj && obj.count(k) > 0; }
  const Json &at(const std::string &k) const {
    auto it = obj.find(k);
    if (type != Obj || it == obj.end()) throw std::runtime_error("json: missing key '" + k + "'");
    return it->second;
  }
  Json &operator[](const std::string &k) {
    type = Obj;
    return obj[k];
  }
  double as_num() const {
    if (type == Num) return num;
    if (type == Bool) return b ? 1.0 : 0.0;
    throw std::runtime_error("json: number expected");
  }
  bool as_bool() const {
    if (type == Bool) return b;
    if (type == Num) return num != 0;
    throw std::runtime_error("json: boolean expected");
  }
};

class JsonParser {
 public:
  explicit JsonParser(const char *s) : p_(s) {}
  Json parse() {
    Json v = value();
    ws();
    if (*p_) fail("trailing characters");
    return v;
  }

 private:
  const char *p_;
  [[noreturn]] void fail(const char *m) { throw std::runtime_error(std::string("json parse error: ") + m); }
  void ws() {
    while (*p_ == ' ' || *p_ == '\t' || *p_ == '\n' || *p_ == '\r') ++p_;
  }
  Json value() {
    ws();
    switch (*p_) {
      case '{': return object();
      case '[': return array();
      case '"': return Json::string(string());
      case 't':
        if (!strncmp(p_, "true", 4)) {
          p_ += 4;
          return Json::boolean(true);
        }
        fail("bad literal");
      case 'f':
        if (!strncmp(p_, "false", 5)) {
          p_ += 5;
          return Json::boolean(false);
        }
        fail("bad literal");
      case 'n':
        if (!strncmp(p_, "null", 4)) {
          p_ += 4;
          return Json();
        }
        fail("bad literal");
      case 'N':  // python's json.dumps writes NaN / Infinity for non-finite floats
        if (!strncmp(p_, "NaN", 3)) {
          p_ += 3;
          return Json::number(NAN);
        }
        fail("bad literal");
      case 'I':
        if (!strncmp(p_, "Infinity", 8)) {
          p_ += 8;
          return Json::number(INFINITY);
        }
        fail("bad literal");
      default: return number();
    }
  }
  Json number() {
    if (!strncmp(p_, "-Infinity", 9)) {
      p_ += 9;
      return Json::number(-INFINITY);
    }
    char *end = nullptr;
    const double v = strtod(p_, &end);
    if (end == p_) fail("value expected");
    bool is_int = true;
    for (const char *q = p_; q < end; ++q)
      if (*q == '.' || *q == 'e' || *q == 'E') is_int = false;
    p_ = end;
    Json j = Json::number(v);
    j.is_int = is_int;
    return j;
  }
  std::string string() {
    std::string out;
    ++p_;
    while (*p_ && *p_ != '"') {
      if (*p_ == '\\') {
        ++p_;
        switch (*p_) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {
            unsigned code = 0;
            for (int i = 1; i <= 4; ++i) {
              const char c = p_[i];
              if (!c) fail("bad \\u escape");
              code = code * 16 + (c <= '9' ? c - '0' : (c | 32) - 'a' + 10);
            }
            p_ += 4;
            if (code < 0x80) {
              out += char(code);
            } else if (code < 0x800) {
              out += char(0xC0 | (code >> 6));
              out += char(0x80 | (code & 0x3F));
            } else {
              out += char(0xE0 | (code >> 12));
              out += char(0x80 | ((code >> 6) & 0x3F));
              out += char(0x80 | (code & 0x3F));
            }
            break;
          }
          default: out += *p_;
        }
        ++p_;
      } else {
        out += *p_++;
      }
    }
    if (*p_ != '"') fail("unterminated string");
    ++p_;
    return out;
  }
  Json array() {
    Json j = Json::array();
    ++p_;
    ws();
    if (*p_ == ']') {
      ++p_;
      return j;
    }
    for (;;) {
      j.arr.push_back(value());
      ws();
      if (*p_ == ',') {
        ++p_;
        continue;
      }
      if (*p_ == ']') {
        ++p_;
        return j;
      }
      fail("',' or ']' expected");
    }
  }
  Json object() {
    Json j = Json::object();
    ++p_;
    ws();
    if (*p_ == '}') {
      ++p_;
      return j;
    }
    for (;;) {
      ws();
      if (*p_ != '"') fail("key expected");
      std::string k = string();
      ws();
      if (*p_ != ':') fail("':' expected");
      ++p_;
      j.obj[k] = value();
      ws();
      if (*p_ == ',') {
        ++p_;
        continue;
      }
      if (*p_ == '}') {
        ++p_;
        return j;
      }
      fail("',' or '}' expected");
    }
  }
};

// shortest decimal text that strtod() maps back to the same double
inline std::string json_double(double v) {
  if (!std::isfinite(v)) return "null";
  char buf[40];
  for (int prec = 1; prec <= 17; ++prec) {
    snprintf(buf, sizeof buf, "%.*g", prec, v);
    if (strtod(buf, nullptr) == v) break;
  }
  std::string s(buf);
  if (s.find_first_of(".eEn") == std::string::npos) s += ".0";
  return s;
}

inline void json_write(const Json &j, std::string &out) {
  switch (j.type) {
    case Json::Null: out += "null"; break;
    case Json::Bool: out += j.b ? "true" : "false"; break;
    case Json::Num:
      if (j.is_int) {
        char buf[32];
        snprintf(buf, sizeof buf, "%lld", (long long)j.num);
        out += buf;
      } else {
        out += json_double(j.num);
      }
      break;
    case Json::Str:
      out += '"';
      for (char c : j.str) {
        if (c == '"' || c == '\\') {
          out += '\\';
          out += c;
        } else if (c == '\n') {
          out += "\\n";
        } else {
          out += c;
        }
      }
      out += '"';
      break;
    case Json::Arr: {
      out += '[';
      bool first = true;
      for (const Json &e : j.arr) {
        if (!first) out += ',';
        first = false;
        json_write(e, out);
      }
      out += ']';
      break;
    }
    case Json::Obj: {
      out += '{';
      bool first = true;
      for (const auto &kv : j.obj) {
        if (!first) out += ',';
        first = false;
        out += '"';
        out += kv.first;
        out += "\":";
        json_write(kv.second, out);
      }
      out += '}';
      break;
    }
  }
}

}  // namespace arb
