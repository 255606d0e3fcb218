// A small strict JSON reader (RFC 8259 numbers, well-formed UTF-8, no control characters or lone surrogates, finite
// numbers) shared by the checkpoint loader and the model-configuration registry.  Header-only, host code.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <utility>
#include <vector>

namespace nvcjson {

// ---------------------------------------------------------------------------------- tiny JSON
struct JValue {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<JValue> arr;
  std::vector<std::pair<std::string, JValue>> obj;   // insertion order kept

  const JValue* get(const std::string& key) const {
    if (kind != Obj) return nullptr;
    for (auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
};

struct JParser {
  const char* p;
  const char* end;
  std::string err;

  bool fail(const std::string& m) {
    if (err.empty()) err = m;
    return false;
  }
  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  bool lit(const char* s) {
    const size_t n = strlen(s);
    if ((size_t)(end - p) < n || memcmp(p, s, n) != 0) return fail(std::string("expected ") + s);
    p += n;
    return true;
  }
  static void utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out += (char)cp;
    else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
  }
  bool hex4(uint32_t& v) {
    if (end - p < 4) return fail("truncated \\u escape");
    v = 0;
    for (int i = 0; i < 4; ++i) {
      const char c = *p++;
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else return fail("bad \\u escape");
    }
    return true;
  }
  bool string(std::string& out) {
    if (p >= end || *p != '"') return fail("expected string");
    ++p;
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (++p >= end) return fail("truncated escape");
        const char c = *p++;
        switch (c) {
          case '"': out += '"'; break;
          case '\\': out += '\\'; break;
          case '/': out += '/'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'n': out += '\n'; break;
          case 'r': out += '\r'; break;
          case 't': out += '\t'; break;
          case 'u': {
            uint32_t cp;
            if (!hex4(cp)) return false;
            if (cp >= 0xDC00 && cp < 0xE000) return fail("lone trailing surrogate in \\u escape");
            if (cp >= 0xD800 && cp < 0xDC00) {
              if (end - p < 6 || p[0] != '\\' || p[1] != 'u') return fail("lone leading surrogate in \\u escape");
              p += 2;
              uint32_t lo;
              if (!hex4(lo)) return false;
              if (lo < 0xDC00 || lo >= 0xE000) return fail("lone leading surrogate in \\u escape");
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            utf8(out, cp);
            break;
          }
          default: return fail("bad escape");
        }
      } else {
        // raw bytes: no control characters, well-formed UTF-8 only (what serde_json / RFC 8259 accept)
        const unsigned char c = (unsigned char)*p;
        if (c < 0x20) return fail("control character in string");
        int extra = 0;
        uint32_t cp = c;
        if (c >= 0x80) {
          if (c >= 0xC2 && c <= 0xDF) { extra = 1; cp = c & 0x1F; }
          else if (c >= 0xE0 && c <= 0xEF) { extra = 2; cp = c & 0x0F; }
          else if (c >= 0xF0 && c <= 0xF4) { extra = 3; cp = c & 0x07; }
          else return fail("invalid UTF-8 in string");
          if (end - p <= extra) return fail("invalid UTF-8 in string");
          for (int i = 1; i <= extra; ++i) {
            const unsigned char cc = (unsigned char)p[i];
            if ((cc & 0xC0) != 0x80) return fail("invalid UTF-8 in string");
            cp = (cp << 6) | (cc & 0x3F);
          }
          if ((extra == 2 && (cp < 0x800 || (cp >= 0xD800 && cp < 0xE000))) || (extra == 3 && (cp < 0x10000 || cp > 0x10FFFF)))
            return fail("invalid UTF-8 in string");
        }
        out.append(p, (size_t)extra + 1);
        p += extra + 1;
      }
    }
    if (p >= end) return fail("unterminated string");
    ++p;
    return true;
  }
  bool value(JValue& v, int depth = 0) {
    if (depth > 64) return fail("nesting too deep");
    ws();
    if (p >= end) return fail("unexpected end of input");
    const char c = *p;
    if (c == '{') {
      v.kind = JValue::Obj;
      ++p;
      ws();
      if (p < end && *p == '}') { ++p; return true; }
      for (;;) {
        ws();
        std::string key;
        if (!string(key)) return false;
        ws();
        if (p >= end || *p != ':') return fail("expected ':'");
        ++p;
        JValue child;
        if (!value(child, depth + 1)) return false;
        v.obj.emplace_back(std::move(key), std::move(child));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == '}') { ++p; return true; }
        return fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      v.kind = JValue::Arr;
      ++p;
      ws();
      if (p < end && *p == ']') { ++p; return true; }
      for (;;) {
        JValue child;
        if (!value(child, depth + 1)) return false;
        v.arr.push_back(std::move(child));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == ']') { ++p; return true; }
        return fail("expected ',' or ']'");
      }
    }
    if (c == '"') { v.kind = JValue::Str; return string(v.str); }
    if (c == 't') { v.kind = JValue::Bool; v.b = true; return lit("true"); }
    if (c == 'f') { v.kind = JValue::Bool; v.b = false; return lit("false"); }
    if (c == 'n') { v.kind = JValue::Null; return lit("null"); }
    // number
    // number: -? (0 | [1-9][0-9]*) (. [0-9]+)? ([eE] [+-]? [0-9]+)?   (RFC 8259)
    const char* s = p;
    auto digits = [&]() { const char* d = p; while (p < end && *p >= '0' && *p <= '9') ++p; return p > d; };
    if (p < end && *p == '-') ++p;
    if (p < end && *p == '0') ++p;
    else if (!digits()) return fail(p == s ? "unexpected character" : "invalid number");
    if (p < end && *p == '.') { ++p; if (!digits()) return fail("invalid number"); }
    if (p < end && (*p == 'e' || *p == 'E')) {
      ++p;
      if (p < end && (*p == '+' || *p == '-')) ++p;
      if (!digits()) return fail("invalid number");
    }
    v.kind = JValue::Num;
    v.num = strtod(std::string(s, p).c_str(), nullptr);
    if (!std::isfinite(v.num)) return fail("number out of range");
    return true;
  }
};

inline bool parse_json(const char* data, size_t n, JValue& out, std::string& err) {
  JParser ps{data, data + n, ""};
  if (!ps.value(out)) { err = ps.err; return false; }
  ps.ws();
  if (ps.p != ps.end) { err = "trailing characters after JSON value"; return false; }
  return true;
}

inline bool read_file(const std::string& path, std::string& out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  std::ostringstream ss;
  ss << f.rdbuf();
  out = ss.str();
  return true;
}


}  // namespace nvcjson
