// json_min.h -- a small JSON document reader (objects, arrays, strings, numbers, true/false/null) for model
// configuration files (config.json) and safetensors headers.  Header-only, no third-party code.  Numbers are kept
// as double; object members keep file order and are looked up linearly (configuration files are small).
#pragma once
#include <stdlib.h>

#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace qie {

struct JsonValue {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<JsonValue> arr;
  std::vector<std::pair<std::string, JsonValue>> obj;

  const JsonValue* get(const char* key) const {
    if (kind != Object) return nullptr;
    for (const auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  // member that is present and not null
  const JsonValue* have(const char* key) const {
    const JsonValue* v = get(key);
    return (v && v->kind != Null) ? v : nullptr;
  }
  bool is_number() const { return kind == Number; }
  double number_or(double dflt) const { return kind == Number ? num : dflt; }
};

class JsonReader {
 public:
  // parses [p, e); returns false and sets err on malformed input
  static bool parse(const char* p, const char* e, JsonValue* out, std::string* err) {
    JsonReader r(p, e);
    if (!r.value(out, 0)) {
      if (err) *err = "json: " + r.err_ + " at byte " + std::to_string((long)(r.p_ - p));
      return false;
    }
    r.ws();
    if (r.p_ != e) {
      if (err) *err = "json: trailing bytes";
      return false;
    }
    return true;
  }

 private:
  JsonReader(const char* p, const char* e) : p_(p), e_(e) {}
  const char* p_;
  const char* e_;
  std::string err_;

  bool fail(const char* m) {
    if (err_.empty()) err_ = m;
    return false;
  }
  void ws() {
    while (p_ < e_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
  }
  bool word(const char* w) {
    const char* q = p_;
    while (*w && q < e_ && *q == *w) ++q, ++w;
    if (*w) return false;
    p_ = q;
    return true;
  }
  bool string(std::string* out) {
    if (p_ >= e_ || *p_ != '"') return fail("expected string");
    ++p_;
    out->clear();
    while (p_ < e_ && *p_ != '"') {
      if (*p_ == '\\') {
        if (++p_ >= e_) return fail("bad escape");
        switch (*p_) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          case 'r': out->push_back('\r'); break;
          case 'b': out->push_back('\b'); break;
          case 'f': out->push_back('\f'); break;
          case 'u': {  // \uXXXX: ASCII range decoded, anything else kept as '?'
            if (e_ - p_ < 5) return fail("bad \\u escape");
            const std::string hex(p_ + 1, p_ + 5);
            const long cp = strtol(hex.c_str(), nullptr, 16);
            out->push_back(cp > 0 && cp < 128 ? (char)cp : '?');
            p_ += 4;
            break;
          }
          default: out->push_back(*p_); break;
        }
        ++p_;
      } else {
        out->push_back(*p_++);
      }
    }
    if (p_ >= e_) return fail("unterminated string");
    ++p_;
    return true;
  }
  bool value(JsonValue* v, int depth) {
    if (depth > 64) return fail("nesting too deep");
    ws();
    if (p_ >= e_) return fail("unexpected end");
    const char c = *p_;
    if (c == '{') {
      ++p_;
      v->kind = JsonValue::Object;
      ws();
      if (p_ < e_ && *p_ == '}') return ++p_, true;
      for (;;) {
        ws();
        std::string k;
        if (!string(&k)) return false;
        ws();
        if (p_ >= e_ || *p_ != ':') return fail("expected ':'");
        ++p_;
        v->obj.emplace_back(std::move(k), JsonValue());
        if (!value(&v->obj.back().second, depth + 1)) return false;
        ws();
        if (p_ < e_ && *p_ == ',') {
          ++p_;
          continue;
        }
        if (p_ < e_ && *p_ == '}') return ++p_, true;
        return fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      ++p_;
      v->kind = JsonValue::Array;
      ws();
      if (p_ < e_ && *p_ == ']') return ++p_, true;
      for (;;) {
        v->arr.emplace_back();
        if (!value(&v->arr.back(), depth + 1)) return false;
        ws();
        if (p_ < e_ && *p_ == ',') {
          ++p_;
          continue;
        }
        if (p_ < e_ && *p_ == ']') return ++p_, true;
        return fail("expected ',' or ']'");
      }
    }
    if (c == '"') {
      v->kind = JsonValue::String;
      return string(&v->str);
    }
    if (word("true")) return v->kind = JsonValue::Bool, v->b = true, true;
    if (word("false")) return v->kind = JsonValue::Bool, v->b = false, true;
    if (word("null")) return v->kind = JsonValue::Null, true;
    {
      const std::string tmp(p_, (size_t)(e_ - p_ < 64 ? e_ - p_ : 64));
      char* end = nullptr;
      const double d = strtod(tmp.c_str(), &end);
      if (end == tmp.c_str()) return fail("expected a value");
      p_ += end - tmp.c_str();
      v->kind = JsonValue::Number;
      v->num = d;
      return true;
    }
  }
};

}  // namespace qie
