#include "json.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

namespace pccl {

namespace {
struct Parser {
  const char* p;
  const char* end;
  int depth = 0;

  [[noreturn]] void fail(const char* what) {
    throw std::runtime_error(std::string("json: ") + what);
  }
  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  bool eat(char c) {
    ws();
    if (p < end && *p == c) { ++p; return true; }
    return false;
  }
  void expect(char c) {
    if (!eat(c)) fail("unexpected character");
  }
  std::string str() {
    std::string out;
    if (p >= end || *p != '"') fail("expected string");
    ++p;
    while (p < end && *p != '"') {
      char c = *p++;
      if (c != '\\') { out.push_back(c); continue; }
      if (p >= end) fail("bad escape");
      char e = *p++;
      switch (e) {
        case 'n': out.push_back('\n'); break;
        case 't': out.push_back('\t'); break;
        case 'r': out.push_back('\r'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'u': {
          if (end - p < 4) fail("bad \\u escape");
          unsigned cp = 0;
          for (int i = 0; i < 4; ++i) {
            char h = *p++;
            cp <<= 4;
            if (h >= '0' && h <= '9') cp |= h - '0';
            else if (h >= 'a' && h <= 'f') cp |= h - 'a' + 10;
            else if (h >= 'A' && h <= 'F') cp |= h - 'A' + 10;
            else fail("bad \\u escape");
          }
          if (cp < 0x80) out.push_back(static_cast<char>(cp));
          else if (cp < 0x800) { out.push_back(0xC0 | (cp >> 6)); out.push_back(0x80 | (cp & 0x3F)); }
          else { out.push_back(0xE0 | (cp >> 12)); out.push_back(0x80 | ((cp >> 6) & 0x3F)); out.push_back(0x80 | (cp & 0x3F)); }
          break;
        }
        default: out.push_back(e);
      }
    }
    if (p >= end) fail("unterminated string");
    ++p;
    return out;
  }
  Json value() {
    if (++depth > 256) fail("nesting too deep");
    ws();
    if (p >= end) fail("unexpected end");
    Json out;
    char c = *p;
    if (c == '{') {
      ++p;
      out = Json::object();
      if (!eat('}')) {
        do {
          ws();
          std::string k = str();
          expect(':');
          out.set(k, value());
        } while (eat(','));
        expect('}');
      }
    } else if (c == '[') {
      ++p;
      out = Json::array();
      if (!eat(']')) {
        do { out.push(value()); } while (eat(','));
        expect(']');
      }
    } else if (c == '"') {
      out = Json(str());
    } else if (!std::strncmp(p, "true", std::min<size_t>(4, end - p)) && end - p >= 4) {
      p += 4; out = Json(true);
    } else if (!std::strncmp(p, "false", std::min<size_t>(5, end - p)) && end - p >= 5) {
      p += 5; out = Json(false);
    } else if (!std::strncmp(p, "null", std::min<size_t>(4, end - p)) && end - p >= 4) {
      p += 4;
    } else {
      const char* s = p;
      bool is_int = true;
      if (p < end && (*p == '-' || *p == '+')) ++p;
      while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '-' || *p == '+')) {
        if (*p == '.' || *p == 'e' || *p == 'E') is_int = false;
        ++p;
      }
      if (p == s) fail("unexpected token");
      std::string num(s, p - s);
      if (is_int) out = Json(static_cast<int64_t>(std::strtoll(num.c_str(), nullptr, 10)));
      else out = Json(std::strtod(num.c_str(), nullptr));
    }
    --depth;
    return out;
  }
};

void escapeTo(std::string& out, const std::string& s) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\t': out += "\\t"; break;
      case '\r': out += "\\r"; break;
      default:
        if (c < 0x20) { char b[8]; std::snprintf(b, sizeof(b), "\\u%04x", c); out += b; }
        else out.push_back(static_cast<char>(c));
    }
  }
  out.push_back('"');
}
}  // namespace

Json Json::parse(const std::string& text) {
  Parser ps{text.data(), text.data() + text.size()};
  Json v = ps.value();
  ps.ws();
  if (ps.p != ps.end) ps.fail("trailing characters");
  return v;
}

Json Json::parseFile(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("json: cannot open " + path);
  std::stringstream ss;
  ss << f.rdbuf();
  return parse(ss.str());
}

void Json::dumpTo(std::string& out) const {
  switch (kind_) {
    case Kind::Null: out += "null"; break;
    case Kind::Bool: out += b_ ? "true" : "false"; break;
    case Kind::Number: {
      char b[40];
      if (is_int_) std::snprintf(b, sizeof(b), "%lld", static_cast<long long>(i_));
      else if (std::isfinite(n_)) std::snprintf(b, sizeof(b), "%.17g", n_);
      else std::snprintf(b, sizeof(b), "null");
      out += b;
      break;
    }
    case Kind::String: escapeTo(out, s_); break;
    case Kind::Array:
      out.push_back('[');
      for (size_t i = 0; i < a_.size(); ++i) { if (i) out.push_back(','); a_[i].dumpTo(out); }
      out.push_back(']');
      break;
    case Kind::Object:
      out.push_back('{');
      for (size_t i = 0; i < o_.size(); ++i) {
        if (i) out.push_back(',');
        escapeTo(out, o_[i].first);
        out.push_back(':');
        o_[i].second.dumpTo(out);
      }
      out.push_back('}');
      break;
  }
}

std::string Json::dump() const {
  std::string out;
  dumpTo(out);
  return out;
}

}  // namespace pccl
