// Minimal JSON value, parser and printer used for marker payloads, per-task
// options and plan / manifest dumps (the role json_utils.h plays in the
// reference, src/pjrt_client/json_utils.h).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace mmg {

class Json {
 public:
  enum Kind { Null, Bool, Number, String, Array, Object };
  Kind kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;

  Json() = default;
  static Json boolean(bool v) { Json j; j.kind = Bool; j.b = v; return j; }
  static Json number(double v) { Json j; j.kind = Number; j.num = v; return j; }
  static Json string(std::string v) { Json j; j.kind = String; j.str = std::move(v); return j; }
  static Json array() { Json j; j.kind = Array; return j; }
  static Json object() { Json j; j.kind = Object; return j; }

  bool is_null() const { return kind == Null; }
  bool is_array() const { return kind == Array; }
  bool is_object() const { return kind == Object; }
  bool is_string() const { return kind == String; }
  bool is_number() const { return kind == Number; }
  int64_t as_int() const { return kind == Bool ? (b ? 1 : 0) : static_cast<int64_t>(num); }
  bool as_bool() const { return kind == Bool ? b : num != 0; }
  const Json* find(const std::string& key) const {
    for (auto& kv : obj) if (kv.first == key) return &kv.second;
    return nullptr;
  }
  bool has(const std::string& key) const { return find(key) != nullptr; }
  const Json& at(const std::string& key) const {
    const Json* j = find(key);
    if (!j) throw std::runtime_error("json: missing key " + key);
    return *j;
  }
  Json& set(const std::string& key, Json v) {
    for (auto& kv : obj) if (kv.first == key) { kv.second = std::move(v); return kv.second; }
    kind = Object;
    obj.emplace_back(key, std::move(v));
    return obj.back().second;
  }
  void push(Json v) { kind = Array; arr.push_back(std::move(v)); }
  size_t size() const { return kind == Array ? arr.size() : obj.size(); }

  std::vector<int64_t> as_int_vector() const {
    std::vector<int64_t> out;
    for (auto& e : arr) out.push_back(e.as_int());
    return out;
  }
  std::vector<std::string> as_string_vector() const {
    std::vector<std::string> out;
    for (auto& e : arr) out.push_back(e.str);
    return out;
  }

  std::string dump() const {
    std::ostringstream os;
    write(os);
    return os.str();
  }
  void write(std::ostream& os) const {
    switch (kind) {
      case Null: os << "null"; break;
      case Bool: os << (b ? "true" : "false"); break;
      case Number:
        if (num == static_cast<double>(static_cast<int64_t>(num))) os << static_cast<int64_t>(num);
        else os << num;
        break;
      case String: write_string(os, str); break;
      case Array:
        os << '[';
        for (size_t i = 0; i < arr.size(); ++i) { if (i) os << ','; arr[i].write(os); }
        os << ']';
        break;
      case Object:
        os << '{';
        for (size_t i = 0; i < obj.size(); ++i) {
          if (i) os << ',';
          write_string(os, obj[i].first);
          os << ':';
          obj[i].second.write(os);
        }
        os << '}';
        break;
    }
  }

  static Json parse(const std::string& text) {
    size_t pos = 0;
    Json j = parse_value(text, pos);
    skip_ws(text, pos);
    if (pos != text.size()) throw std::runtime_error("json: trailing characters");
    return j;
  }

 private:
  static void write_string(std::ostream& os, const std::string& s) {
    os << '"';
    for (char c : s) {
      switch (c) {
        case '"': os << "\\\""; break;
        case '\\': os << "\\\\"; break;
        case '\n': os << "\\n"; break;
        case '\t': os << "\\t"; break;
        default: os << c;
      }
    }
    os << '"';
  }
  static void skip_ws(const std::string& t, size_t& p) {
    while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\t' || t[p] == '\r')) ++p;
  }
  // The character at `p`; text that ends where a character is needed is an error, never a read
  // past the end.
  static char peek(const std::string& t, size_t p) {
    if (p >= t.size()) throw std::runtime_error("json: unexpected end");
    return t[p];
  }
  static constexpr int kMaxDepth = 256;
  static Json parse_value(const std::string& t, size_t& p, int depth = 0) {
    if (depth > kMaxDepth) throw std::runtime_error("json: nested too deeply");
    skip_ws(t, p);
    const char c = peek(t, p);
    if (c == '{') {
      Json j = object();
      ++p;
      skip_ws(t, p);
      if (peek(t, p) == '}') { ++p; return j; }
      while (true) {
        skip_ws(t, p);
        Json key = parse_string(t, p);
        skip_ws(t, p);
        if (peek(t, p) != ':') throw std::runtime_error("json: expected ':'");
        ++p;
        j.obj.emplace_back(key.str, parse_value(t, p, depth + 1));
        skip_ws(t, p);
        const char sep = peek(t, p);
        if (sep == ',') { ++p; continue; }
        if (sep == '}') { ++p; break; }
        throw std::runtime_error("json: expected ',' or '}'");
      }
      return j;
    }
    if (c == '[') {
      Json j = array();
      ++p;
      skip_ws(t, p);
      if (peek(t, p) == ']') { ++p; return j; }
      while (true) {
        j.arr.push_back(parse_value(t, p, depth + 1));
        skip_ws(t, p);
        const char sep = peek(t, p);
        if (sep == ',') { ++p; continue; }
        if (sep == ']') { ++p; break; }
        throw std::runtime_error("json: expected ',' or ']'");
      }
      return j;
    }
    if (c == '"') return parse_string(t, p);
    if (t.compare(p, 4, "true") == 0) { p += 4; return boolean(true); }
    if (t.compare(p, 5, "false") == 0) { p += 5; return boolean(false); }
    if (t.compare(p, 4, "null") == 0) { p += 4; return Json(); }
    size_t end = p;
    while (end < t.size() && (isdigit(static_cast<unsigned char>(t[end])) || t[end] == '-' || t[end] == '+' ||
                              t[end] == '.' || t[end] == 'e' || t[end] == 'E'))
      ++end;
    if (end == p) throw std::runtime_error("json: unexpected character");
    double value = 0;
    try {
      size_t used = 0;
      value = std::stod(t.substr(p, end - p), &used);
      if (used != end - p) throw std::runtime_error("");
    } catch (const std::exception&) {
      throw std::runtime_error("json: malformed number '" + t.substr(p, end - p) + "'");
    }
    p = end;
    return number(value);
  }
  static Json parse_string(const std::string& t, size_t& p) {
    if (peek(t, p) != '"') throw std::runtime_error("json: expected string");
    ++p;
    std::string out;
    while (true) {
      const char c = peek(t, p);      // an unterminated string runs into the end of the text: error
      if (c == '"') break;
      if (c == '\\') {
        ++p;
        const char e = peek(t, p);
        switch (e) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          default: out += e;
        }
      } else {
        out += c;
      }
      ++p;
    }
    ++p;
    return string(out);
  }
};

}  // namespace mmg
