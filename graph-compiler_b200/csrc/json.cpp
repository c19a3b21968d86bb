#include "json.h"

#include <cerrno>
#include <cmath>
#include <cstdlib>

namespace gcb {
namespace {

struct Parser {
  const std::string &s;
  size_t i = 0;
  int depth = 0;
  explicit Parser(const std::string &t) : s(t) {}

  [[noreturn]] void fail(const char *msg) const {
    throw JsonError(std::string("JSON: ") + msg + " at offset " + std::to_string(i));
  }
  void ws() {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\t' || s[i] == '\n' || s[i] == '\r')) ++i;
  }
  bool eat(char c) {
    ws();
    if (i < s.size() && s[i] == c) { ++i; return true; }
    return false;
  }
  void expect(char c) {
    if (!eat(c)) fail("unexpected character");
  }
  JsonValue value() {
    ws();
    if (i >= s.size()) fail("unexpected end of input");
    if (++depth > 64) fail("nesting too deep");
    JsonValue v;
    const char c = s[i];
    if (c == '{') v = object();
    else if (c == '[') v = array();
    else if (c == '"') { v.kind = JsonValue::String; v.str = string(); }
    else if (c == 't' || c == 'f' || c == 'n') v = literal();
    else v = number();
    --depth;
    return v;
  }
  JsonValue object() {
    JsonValue v;
    v.kind = JsonValue::Object;
    expect('{');
    if (eat('}')) return v;
    do {
      ws();
      if (i >= s.size() || s[i] != '"') fail("object key expected");
      std::string k = string();
      expect(':');
      v.obj.emplace_back(std::move(k), value());
    } while (eat(','));
    expect('}');
    return v;
  }
  JsonValue array() {
    JsonValue v;
    v.kind = JsonValue::Array;
    expect('[');
    if (eat(']')) return v;
    do v.arr.push_back(value()); while (eat(','));
    expect(']');
    return v;
  }
  std::string string() {
    std::string out;
    ++i; // opening quote
    while (i < s.size() && s[i] != '"') {
      char c = s[i++];
      if (c == '\\') {
        if (i >= s.size()) fail("bad escape");
        char e = s[i++];
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
          if (i + 4 > s.size()) fail("bad \\u escape");
          unsigned cp = unsigned(std::strtoul(s.substr(i, 4).c_str(), nullptr, 16));
          i += 4;
          if (cp < 0x80) out += char(cp);
          else if (cp < 0x800) { out += char(0xC0 | (cp >> 6)); out += char(0x80 | (cp & 0x3F)); }
          else { out += char(0xE0 | (cp >> 12)); out += char(0x80 | ((cp >> 6) & 0x3F)); out += char(0x80 | (cp & 0x3F)); }
          break;
        }
        default: fail("bad escape");
        }
      } else {
        out += c;
      }
    }
    if (i >= s.size()) fail("unterminated string");
    ++i; // closing quote
    return out;
  }
  JsonValue literal() {
    JsonValue v;
    if (s.compare(i, 4, "true") == 0) { v.kind = JsonValue::Bool; v.b = true; i += 4; }
    else if (s.compare(i, 5, "false") == 0) { v.kind = JsonValue::Bool; v.b = false; i += 5; }
    else if (s.compare(i, 4, "null") == 0) { v.kind = JsonValue::Null; i += 4; }
    else fail("bad literal");
    return v;
  }
  JsonValue number() {
    const size_t st = i;
    if (i < s.size() && (s[i] == '-' || s[i] == '+')) ++i;
    bool integer = true;
    while (i < s.size() && (std::isdigit((unsigned char)s[i]) || s[i] == '.' || s[i] == 'e' || s[i] == 'E' ||
                            s[i] == '-' || s[i] == '+')) {
      if (s[i] == '.' || s[i] == 'e' || s[i] == 'E') integer = false;
      ++i;
    }
    if (i == st) fail("value expected");
    const std::string tok = s.substr(st, i - st);
    JsonValue v;
    v.kind = JsonValue::Number;
    char *end = nullptr;
    v.num = std::strtod(tok.c_str(), &end);
    if (end == tok.c_str() || *end != '\0') fail("bad number");
    if (integer) {
      errno = 0;
      long long ll = std::strtoll(tok.c_str(), &end, 10);
      if (errno == 0 && *end == '\0') { v.is_int = true; v.inum = ll; }
    }
    return v;
  }
};

} // namespace

JsonValue parse_json(const std::string &text) {
  Parser p(text);
  JsonValue v = p.value();
  p.ws();
  if (p.i != text.size()) p.fail("trailing characters");
  return v;
}

} // namespace gcb
