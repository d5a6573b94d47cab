// Recursive-descent reader and printer for the fixture subset (see tcrv/Fixture.h).
#include "tcrv/Fixture.h"

#include <cctype>
#include <set>
#include <sstream>

namespace tcrv {

const Attr *Op::attr(const std::string &key) const {
  for (const auto &kv : attrs)
    if (kv.first == key)
      return &kv.second;
  return nullptr;
}

std::string Op::strAttr(const std::string &key) const {
  const Attr *a = attr(key);
  return (a && a->kind == Attr::String) ? a->str : std::string();
}

bool Op::intAttr(const std::string &key, long long &out) const {
  const Attr *a = attr(key);
  if (!a || a->kind != Attr::Integer)
    return false;
  out = a->integer;
  return true;
}

const Op *Op::firstChild(const std::string &opName) const {
  for (const auto &c : body)
    if (c->name == opName)
      return c.get();
  return nullptr;
}

std::vector<const Op *> Op::children(const std::string &opName) const {
  std::vector<const Op *> out;
  for (const auto &c : body)
    if (c->name == opName)
      out.push_back(c.get());
  return out;
}

namespace {

const std::set<std::string> &regionOps() {
  static const std::set<std::string> s = {"module", "tcrv.exec.kernel", "tcrv.exec.variant", "tcrv.exec.dispatch",
                                          "tcrv_rvv.with_vl"};
  return s;
}

struct Parser {
  const std::string &src;
  size_t pos = 0;
  int line = 1;
  std::string error;

  explicit Parser(const std::string &s) : src(s) {}

  bool fail(const std::string &msg) {
    if (error.empty())
      error = "line " + std::to_string(line) + ": " + msg;
    return false;
  }
  bool eof() const { return pos >= src.size(); }
  char peek() const { return eof() ? '\0' : src[pos]; }
  void bump() {
    if (src[pos] == '\n')
      ++line;
    ++pos;
  }
  // skips blanks and `//` comments; stops at a newline when `stopAtNewline`
  void skip(bool stopAtNewline = false) {
    while (!eof()) {
      char c = peek();
      if (c == '\n' && stopAtNewline)
        return;
      if (std::isspace(static_cast<unsigned char>(c))) {
        bump();
      } else if (c == '/' && pos + 1 < src.size() && src[pos + 1] == '/') {
        while (!eof() && peek() != '\n')
          bump();
      } else {
        return;
      }
    }
  }
  bool consume(char c) {
    skip();
    if (peek() != c)
      return false;
    bump();
    return true;
  }
  static bool identChar(char c) { return std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '.' || c == '$' || c == '-'; }
  std::string ident() {
    skip();
    std::string out;
    while (!eof() && identChar(peek())) {
      out.push_back(peek());
      bump();
    }
    return out;
  }
  bool startsWith(const char *kw) {
    skip();
    size_t n = std::char_traits<char>::length(kw);
    if (src.compare(pos, n, kw) != 0)
      return false;
    char after = pos + n < src.size() ? src[pos + n] : '\0';
    return !identChar(after);
  }

  bool parseString(Attr &a) {
    std::string raw = "\"", val;
    bump();  // opening quote
    while (!eof() && peek() != '"') {
      if (peek() == '\\' && pos + 1 < src.size()) {
        raw.push_back(peek());
        bump();
      }
      raw.push_back(peek());
      val.push_back(peek());
      bump();
    }
    if (eof())
      return fail("unterminated string");
    bump();
    raw.push_back('"');
    a.kind = Attr::String;
    a.text = raw;
    a.str = val;
    return true;
  }

  bool parseAttrValue(Attr &a) {
    skip();
    char c = peek();
    if (c == '"')
      return parseString(a);
    if (c == '[') {
      bump();
      a.kind = Attr::Array;
      a.text = "[";
      skip();
      if (peek() == ']') {
        bump();
        a.text = "[]";
        return true;
      }
      while (true) {
        Attr e;
        if (!parseAttrValue(e))
          return false;
        if (a.elements.size())
          a.text += ", ";
        a.text += e.text;
        a.elements.push_back(e);
        if (consume(','))
          continue;
        if (consume(']'))
          break;
        return fail("expected ',' or ']' in array attribute");
      }
      a.text += "]";
      return true;
    }
    if (c == '@') {
      bump();
      a.kind = Attr::SymbolRef;
      a.str = ident();
      a.text = "@" + a.str;
      return !a.str.empty() || fail("empty symbol reference");
    }
    if (std::isdigit(static_cast<unsigned char>(c)) || c == '-') {
      std::string num;
      num.push_back(c);
      bump();
      while (!eof() && std::isdigit(static_cast<unsigned char>(peek()))) {
        num.push_back(peek());
        bump();
      }
      a.kind = Attr::Integer;
      a.integer = std::stoll(num);
      a.text = num;
      skip(true);
      if (peek() == ':') {  // typed integer, e.g. `32 : i64`
        bump();
        std::string ty = ident();
        if (ty.empty())
          return fail("expected a type after ':' in integer attribute");
        a.text += " : " + ty;
      }
      return true;
    }
    // opaque: dialect attribute (#tcrv_rvv.policy<...>) or a bare word
    int angle = 0;
    std::string raw;
    while (!eof()) {
      char d = peek();
      if (d == '<')
        ++angle;
      if (d == '>')
        --angle;
      if (angle == 0 && (d == ',' || d == '}' || d == ']' || d == '\n'))
        break;
      raw.push_back(d);
      bump();
    }
    while (!raw.empty() && std::isspace(static_cast<unsigned char>(raw.back())))
      raw.pop_back();
    if (raw.empty())
      return fail("expected an attribute value");
    a.kind = Attr::Opaque;
    a.text = raw;
    return true;
  }

  bool parseAttrDict(Op &op) {
    if (!consume('{'))
      return fail("expected '{' to open an attribute dictionary");
    if (consume('}'))
      return true;
    while (true) {
      std::string key = ident();
      if (key.empty())
        return fail("expected an attribute name");
      if (!consume('='))
        return fail("expected '=' after attribute name '" + key + "'");
      Attr a;
      if (!parseAttrValue(a))
        return false;
      if (op.attr(key))
        return fail("duplicate attribute '" + key + "'");
      op.attrs.emplace_back(key, a);
      if (consume(','))
        continue;
      if (consume('}'))
        return true;
      return fail("expected ',' or '}' in attribute dictionary");
    }
  }

  static std::vector<std::string> splitTypes(const std::string &s) {
    std::vector<std::string> out;
    std::string cur;
    int depth = 0;
    bool inStr = false;
    for (char c : s) {
      if (c == '"')
        inStr = !inStr;
      if (!inStr) {
        if (c == '<' || c == '(')
          ++depth;
        if (c == '>' || c == ')')
          --depth;
        if (c == ',' && depth == 0) {
          out.push_back(cur);
          cur.clear();
          continue;
        }
      }
      cur.push_back(c);
    }
    out.push_back(cur);
    std::vector<std::string> trimmed;
    for (auto &t : out) {
      size_t b = t.find_first_not_of(" \t"), e = t.find_last_not_of(" \t");
      if (b != std::string::npos)
        trimmed.push_back(t.substr(b, e - b + 1));
    }
    return trimmed;
  }

  void parseTypeSignature(Op &op) {
    std::string rest;
    while (!eof() && peek() != '\n') {
      if (peek() == '/' && pos + 1 < src.size() && src[pos + 1] == '/')
        break;
      rest.push_back(peek());
      bump();
    }
    // top-level "->" (never inside <...> in these fixtures)
    size_t arrow = std::string::npos;
    int depth = 0;
    for (size_t i = 0; i + 1 < rest.size(); ++i) {
      if (rest[i] == '<')
        ++depth;
      else if (rest[i] == '>' && (i == 0 || rest[i - 1] != '-'))
        --depth;
      if (depth == 0 && rest[i] == '-' && rest[i + 1] == '>') {
        arrow = i;
        break;
      }
    }
    if (arrow != std::string::npos) {
      op.operandTypes = splitTypes(rest.substr(0, arrow));
      op.resultTypes = splitTypes(rest.substr(arrow + 2));
    } else if (!op.results.empty() && op.operands.empty()) {
      op.resultTypes = splitTypes(rest);
    } else {
      op.operandTypes = splitTypes(rest);
    }
  }

  bool parseRegion(Op &op) {
    if (!consume('{'))
      return fail("expected '{' to open a region");
    op.hasRegion = true;
    while (true) {
      skip();
      if (eof())
        return fail("unterminated region of '" + op.name + "'");
      if (peek() == '}') {
        bump();
        return true;
      }
      auto child = std::make_unique<Op>();
      if (!parseOp(*child))
        return false;
      op.body.push_back(std::move(child));
    }
  }

  bool parseOp(Op &op) {
    skip();
    op.line = line;
    if (peek() == '%') {
      while (true) {
        skip();
        if (peek() != '%')
          return fail("expected an SSA result name");
        bump();
        op.results.push_back("%" + ident());
        if (consume(','))
          continue;
        if (consume('='))
          break;
        return fail("expected '=' after result list");
      }
    }
    op.name = ident();
    if (op.name.empty())
      return fail("expected an operation name");
    const bool holdsRegion = regionOps().count(op.name) != 0;
    skip(true);
    if (peek() == '@') {
      bump();
      op.symbol = ident();
    }
    // operands
    skip(true);
    while (peek() == '%') {
      bump();
      op.operands.push_back("%" + ident());
      skip(true);
      if (peek() == ',') {
        bump();
        skip();
      } else {
        break;
      }
    }
    bool sawAttributesKw = false;
    if (startsWith("attributes")) {
      pos += 10;
      sawAttributesKw = true;
    }
    skip(true);
    if (peek() == '{') {
      if (!holdsRegion || sawAttributesKw) {
        if (!parseAttrDict(op))
          return false;
        skip(true);
        if (holdsRegion && peek() == '{' && !parseRegion(op))
          return false;
      } else if (!parseRegion(op)) {
        return false;
      }
    }
    skip(true);
    if (peek() == ':') {
      bump();
      parseTypeSignature(op);
    }
    return true;
  }
};

void printAttrs(std::ostringstream &os, const Op &op) {
  os << "{";
  bool first = true;
  for (const auto &kv : op.attrs) {
    if (!first)
      os << ", ";
    first = false;
    os << kv.first << " = " << kv.second.text;
  }
  os << "}";
}

std::string joinTypes(const std::vector<std::string> &v) {
  std::string out;
  for (size_t i = 0; i < v.size(); ++i)
    out += (i ? ", " : "") + v[i];
  return out;
}

}  // namespace

ParseResult parseFixture(const std::string &text) {
  ParseResult r;
  Parser p(text);
  auto op = std::make_unique<Op>();
  if (!p.parseOp(*op)) {
    r.error = p.error;
    return r;
  }
  if (op->name != "module") {
    r.error = "line " + std::to_string(op->line) + ": expected a top-level 'module'";
    return r;
  }
  p.skip();
  if (!p.eof()) {
    p.fail("unexpected text after the module");
    r.error = p.error;
    return r;
  }
  r.module = std::move(op);
  return r;
}

std::string printOp(const Op &op, int indent) {
  std::ostringstream os;
  const std::string pad(indent, ' ');
  os << pad;
  for (size_t i = 0; i < op.results.size(); ++i)
    os << (i ? ", " : "") << op.results[i];
  if (!op.results.empty())
    os << " = ";
  os << op.name;
  if (!op.symbol.empty())
    os << " @" << op.symbol;
  for (size_t i = 0; i < op.operands.size(); ++i)
    os << (i ? ", " : " ") << op.operands[i];
  if (!op.attrs.empty()) {
    os << (op.hasRegion ? " attributes " : " ");
    printAttrs(os, op);
  }
  if (op.hasRegion) {
    os << " {\n";
    for (const auto &c : op.body)
      os << printOp(*c, indent + 2);
    os << pad << "}";
  }
  if (!op.operandTypes.empty() || !op.resultTypes.empty()) {
    os << " : " << joinTypes(op.operandTypes);
    if (!op.resultTypes.empty())
      os << (op.operandTypes.empty() ? "" : " -> ") << joinTypes(op.resultTypes);
  }
  os << "\n";
  return os.str();
}

}  // namespace tcrv
