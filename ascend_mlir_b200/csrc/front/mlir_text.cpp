#include "front/mlir_text.h"

#include <algorithm>
#include <cctype>
#include <cstdlib>

namespace afir {
namespace front {

std::string Type::str() const {
  if (!isTensor) return elem;
  std::string s = "tensor<";
  for (int64_t d : dims) s += (d < 0 ? std::string("?") : std::to_string(d)) + "x";
  return s + elem + ">";
}

std::string AffineMap::str() const {
  std::string s = "affine_map<(";
  for (int i = 0; i < numDims; ++i) s += (i ? ", d" : "d") + std::to_string(i);
  s += ") -> (";
  for (size_t i = 0; i < results.size(); ++i)
    s += (i ? ", " : "") + (results[i] < 0 ? std::string("0") : "d" + std::to_string(results[i]));
  return s + ")>";
}

namespace {

class Parser {
public:
  Parser(const std::string &text, Module &m) : s_(text), m_(m) {}

  Status run() {
    m_.source = s_;
    skip();
    while (!eof()) {
      if (peek() == '#') {
        if (Status st = mapAlias(); !st) return st;
      } else if (lookingAt("module")) {
        pos_ += 6;
        skip();
        if (lookingAt("attributes")) {
          m_.moduleAttrBegin = pos_;
          pos_ += 10;
          skip();
          if (Status st = skipBalanced('{', '}'); !st) return st;
          m_.moduleAttrEnd = pos_;
          skip();
        }
        if (Status st = expect('{'); !st) return st;
        moduleDepth_ += 1;
      } else if (peek() == '}' && moduleDepth_ > 0) {
        ++pos_;
        moduleDepth_ -= 1;
      } else if (lookingAt("func.func")) {
        if (Status st = func(); !st) return st;
      } else if (lookingAt("transform.named_sequence")) {
        if (Status st = namedSequence(); !st) return st;
      } else {
        return fail("expected 'module', 'func.func', 'transform.named_sequence' or an affine_map alias");
      }
      skip();
    }
    if (moduleDepth_ != 0) return fail("unterminated module");
    return Status::success();
  }

private:
  const std::string &s_;
  Module &m_;
  size_t pos_ = 0;
  int moduleDepth_ = 0;
  int regionDepth_ = 0;  // linalg.generic bodies being parsed (a body that holds another generic, and so on)

  bool eof() const { return pos_ >= s_.size(); }
  char peek() const { return eof() ? '\0' : s_[pos_]; }
  int lineOf(size_t p) const { return 1 + static_cast<int>(std::count(s_.begin(), s_.begin() + std::min(p, s_.size()), '\n')); }
  Status fail(const std::string &msg) const { return Status::error("line " + std::to_string(lineOf(pos_)) + ": " + msg); }

  void skip() {
    while (!eof()) {
      const char c = s_[pos_];
      if (c == ' ' || c == '\t' || c == '\n' || c == '\r') ++pos_;
      else if (c == '/' && pos_ + 1 < s_.size() && s_[pos_ + 1] == '/') {
        while (!eof() && s_[pos_] != '\n') ++pos_;
      } else break;
    }
  }
  bool lookingAt(const char *word) const {
    const size_t n = std::char_traits<char>::length(word);
    if (s_.compare(pos_, n, word) != 0) return false;
    const char next = pos_ + n < s_.size() ? s_[pos_ + n] : '\0';
    return !(std::isalnum(static_cast<unsigned char>(next)) || next == '_' || next == '.');
  }
  bool accept(char c) {
    skip();
    if (peek() == c) { ++pos_; return true; }
    return false;
  }
  bool acceptWord(const char *w) {
    skip();
    if (!lookingAt(w)) return false;
    pos_ += std::char_traits<char>::length(w);
    return true;
  }
  Status expect(char c) {
    skip();
    if (peek() != c) return fail(std::string("expected '") + c + "'");
    ++pos_;
    return Status::success();
  }
  Status expectWord(const char *w) {
    if (!acceptWord(w)) return fail(std::string("expected '") + w + "'");
    return Status::success();
  }
  Status skipBalanced(char open, char close) {
    skip();
    if (peek() != open) return fail(std::string("expected '") + open + "'");
    int depth = 0;
    while (!eof()) {
      const char c = s_[pos_++];
      if (c == '"') {
        while (!eof() && s_[pos_] != '"') pos_ += s_[pos_] == '\\' ? 2 : 1;
        if (eof()) { pos_ = s_.size(); return fail("unterminated string"); }
        ++pos_;
      } else if (c == open) ++depth;
      else if (c == close && --depth == 0) return Status::success();
    }
    return fail("unbalanced brackets");
  }
  std::string ident() {  // bare identifier with dots: linalg.generic, d0, parallel
    skip();
    const size_t b = pos_;
    while (!eof() && (std::isalnum(static_cast<unsigned char>(s_[pos_])) || s_[pos_] == '_' || s_[pos_] == '.' || s_[pos_] == '$')) ++pos_;
    return s_.substr(b, pos_ - b);
  }
  Status ssa(std::string &out) {  // %name
    skip();
    if (peek() != '%') return fail("expected an SSA value");
    ++pos_;
    const size_t b = pos_;
    while (!eof() && (std::isalnum(static_cast<unsigned char>(s_[pos_])) || s_[pos_] == '_' || s_[pos_] == '.' || s_[pos_] == '$' || s_[pos_] == '-')) ++pos_;
    if (pos_ == b) return fail("empty SSA name");
    out = s_.substr(b, pos_ - b);
    return Status::success();
  }
  Status integer(int64_t &out) {
    skip();
    const size_t b = pos_;
    if (peek() == '-' || peek() == '+') ++pos_;
    while (!eof() && std::isdigit(static_cast<unsigned char>(s_[pos_]))) ++pos_;
    if (pos_ == b || (pos_ == b + 1 && !std::isdigit(static_cast<unsigned char>(s_[b])))) return fail("expected an integer");
    out = std::strtoll(s_.substr(b, pos_ - b).c_str(), nullptr, 10);
    return Status::success();
  }

  Status type(Type &t) {
    skip();
    t = Type();
    if (lookingAt("tensor") || lookingAt("memref")) {
      pos_ += 6;
      if (Status st = expect('<'); !st) return st;
      t.isTensor = true;
      while (true) {
        skip();
        if (peek() == '?') {
          ++pos_;
          t.dims.push_back(-1);
        } else if (std::isdigit(static_cast<unsigned char>(peek()))) {
          const size_t b = pos_;
          while (std::isdigit(static_cast<unsigned char>(peek()))) ++pos_;
          t.dims.push_back(std::strtoll(s_.substr(b, pos_ - b).c_str(), nullptr, 10));
        } else break;
        if (peek() != 'x') return fail("expected 'x' in a tensor shape");
        ++pos_;
      }
      t.elem = ident();
      if (t.elem.empty()) return fail("expected an element type");
      return expect('>');
    }
    t.elem = ident();
    if (t.elem.empty()) return fail("expected a type");
    return Status::success();
  }

  Status affineMapBody(AffineMap &map) {  // after "affine_map"
    if (Status st = expect('<'); !st) return st;
    if (Status st = expect('('); !st) return st;
    std::vector<std::string> dims;
    if (!accept(')')) {
      do { dims.push_back(ident()); } while (accept(','));
      if (Status st = expect(')'); !st) return st;
    }
    map.numDims = static_cast<int>(dims.size());
    skip();
    if (s_.compare(pos_, 2, "->") != 0) return fail("expected '->' in an affine map");
    pos_ += 2;
    if (Status st = expect('('); !st) return st;
    if (!accept(')')) {
      do {
        skip();
        if (std::isdigit(static_cast<unsigned char>(peek()))) {
          int64_t c;
          if (Status st = integer(c); !st) return st;
          if (c != 0) return fail("only the constant 0 is supported in indexing maps");
          map.results.push_back(-1);
        } else {
          const std::string d = ident();
          auto it = std::find(dims.begin(), dims.end(), d);
          if (it == dims.end()) return fail("indexing maps must be projected permutations (got '" + d + "')");
          map.results.push_back(static_cast<int>(it - dims.begin()));
        }
      } while (accept(','));
      if (Status st = expect(')'); !st) return st;
    }
    return expect('>');
  }

  Status mapAlias() {  // #name = affine_map<...>
    ++pos_;
    const std::string name = ident();
    if (Status st = expect('='); !st) return st;
    if (!acceptWord("affine_map")) return fail("only affine_map attribute aliases are supported");
    AffineMap map;
    if (Status st = affineMapBody(map); !st) return st;
    m_.mapAliases[name] = map;
    return Status::success();
  }

  Status mapRef(AffineMap &map) {  // #alias or inline affine_map<...>
    skip();
    if (peek() == '#') {
      ++pos_;
      const std::string name = ident();
      auto it = m_.mapAliases.find(name);
      if (it == m_.mapAliases.end()) return fail("unknown affine map alias '#" + name + "'");
      map = it->second;
      return Status::success();
    }
    if (!acceptWord("affine_map")) return fail("expected an affine map");
    return affineMapBody(map);
  }

  Status indexOperand(IndexOperand &io) {
    skip();
    if (peek() == '%') {
      io.literal = false;
      return ssa(io.ssa);
    }
    io.literal = true;
    return integer(io.value);
  }
  Status indexList(std::vector<IndexOperand> &out) {  // [a, b, ...]
    if (Status st = expect('['); !st) return st;
    if (accept(']')) return Status::success();
    do {
      IndexOperand io;
      if (Status st = indexOperand(io); !st) return st;
      out.push_back(io);
    } while (accept(','));
    return expect(']');
  }
  Status ssaList(std::vector<std::string> &out) {
    do {
      std::string v;
      if (Status st = ssa(v); !st) return st;
      out.push_back(v);
    } while (accept(','));
    return Status::success();
  }
  Status typeList(std::vector<Type> &out) {
    do {
      Type t;
      if (Status st = type(t); !st) return st;
      out.push_back(t);
    } while (accept(','));
    return Status::success();
  }

  // transform.named_sequence @name(%root : !transform.any_op {transform.readonly}) { ... }: the region is kept as
  // text; the counts and names this backend uses are picked out of it.
  Status namedSequence() {
    TransformSchedule sched;
    sched.srcBegin = pos_;
    pos_ += std::char_traits<char>::length("transform.named_sequence");
    skip();
    if (peek() != '@') return fail("expected the sequence's symbol name");
    ++pos_;
    sched.name = ident();
    if (Status st = skipBalanced('(', ')'); !st) return st;
    skip();
    if (s_.compare(pos_, 2, "->") == 0) {  // result types
      pos_ += 2;
      if (Status st = skipBalanced('(', ')'); !st) return st;
      skip();
    }
    if (lookingAt("attributes")) { pos_ += 10; if (Status st = skipBalanced('{', '}'); !st) return st; }
    const size_t bodyBegin = pos_;
    if (Status st = skipBalanced('{', '}'); !st) return st;
    sched.srcEnd = pos_;
    const std::string body = s_.substr(bodyBegin, pos_ - bodyBegin);
    if (body.find("transform.yield") == std::string::npos) return fail("transform.named_sequence without a transform.yield");
    auto skipComment = [&](size_t at) {  // true when `at` lies in a // comment
      const size_t lineStart = body.rfind('\n', at);
      const size_t from = lineStart == std::string::npos ? 0 : lineStart;
      const size_t slashes = body.find("//", from);
      return slashes != std::string::npos && slashes < at;
    };
    for (size_t at = body.find("transform.func.add_index_args"); at != std::string::npos; at = body.find("transform.func.add_index_args", at + 1)) {
      if (skipComment(at)) continue;
      const size_t comma = body.find(',', at);
      if (comma == std::string::npos) return fail("transform.func.add_index_args: expected '<function handle>, <count>'");
      const long n = std::strtol(body.c_str() + comma + 1, nullptr, 10);
      if (n <= 0) return fail("transform.func.add_index_args: number of arguments to add must be positive");
      sched.indexArgs += static_cast<int>(n);
    }
    for (size_t at = body.find("tile_sizes"); at != std::string::npos; at = body.find("tile_sizes", at + 1)) {
      if (skipComment(at)) continue;
      const size_t open = body.find('[', at), close = open == std::string::npos ? open : body.find(']', open);
      if (close == std::string::npos) return fail("tile_sizes: expected a bracketed list");
      sched.tileSizes.push_back(body.substr(open, close - open + 1));
    }
    for (size_t at = body.find("transform.annotate"); at != std::string::npos; at = body.find("transform.annotate", at + 1)) {
      if (skipComment(at)) continue;
      const size_t open = body.find('"', at), close = open == std::string::npos ? open : body.find('"', open + 1);
      if (close != std::string::npos) sched.annotations.push_back(body.substr(open + 1, close - open - 1));
    }
    m_.schedules.push_back(std::move(sched));
    return Status::success();
  }

  Status func();
  Status op(Op &o, bool inBody);
  Status generic(Op &o);
  std::string unitIn(size_t from) const;
  std::string unitInDict(size_t begin, size_t end) const;
  Status opList(std::vector<Op> &ops, bool inBody);
};

#include "front/mlir_text_ops.inc"

} // namespace

Status parseModule(const std::string &text, Module &out) {
  out = Module();
  Parser p(text, out);
  return p.run();
}

std::string printModule(const Module &m) {
  // collect insertions (position -> text), then splice from the back
  std::vector<std::pair<size_t, std::string>> ins;
  auto attrText = [](const std::vector<std::pair<std::string, std::string>> &attrs) {
    std::string s;
    for (size_t i = 0; i < attrs.size(); ++i) s += (i ? ", " : "") + attrs[i].first + " = " + attrs[i].second;
    return s;
  };
  for (const Func &f : m.funcs) {
    // attributes the function already carries (from an earlier run over the same text) are not repeated;
    // new ones join the existing dictionary instead of opening a second one
    std::vector<std::pair<std::string, std::string>> fresh;
    for (const auto &kv : f.addedAttrs) {
      bool dup = f.existingAttrs.find(kv.first + " =") != std::string::npos;
      for (const auto &seen : fresh) dup = dup || seen.first == kv.first;
      if (!dup) fresh.push_back(kv);
    }
    if (!fresh.empty() && f.attrDictPos) {
      const bool emptyDict = f.existingAttrs.find_first_not_of("{} \t\n") == std::string::npos;
      ins.emplace_back(f.attrDictPos + 1, attrText(fresh) + (emptyDict ? "" : ", "));
    } else if (!fresh.empty() && f.attrInsertPos) {
      ins.emplace_back(f.attrInsertPos, "attributes {" + attrText(fresh) + "} ");
    }
    for (const Op &o : f.ops) {
      if (o.addedAttrs.empty() || !o.attrInsertPos) continue;
      const bool generic = o.name == "linalg.generic";
      ins.emplace_back(o.attrInsertPos, generic ? "attrs = {" + attrText(o.addedAttrs) + "} " : "{" + attrText(o.addedAttrs) + "} ");
    }
  }
  // erasures are spans [begin, end) replaced by nothing; they never overlap an insertion point
  struct Edit { size_t at; size_t erase; std::string text; };
  std::vector<Edit> edits;
  for (const auto &i : ins) edits.push_back({i.first, 0, i.second});
  for (const auto &e : m.erasures)
    if (e.second > e.first && e.second <= m.source.size()) edits.push_back({e.first, e.second - e.first, std::string()});
  for (const auto &r : m.replacements)
    if (r.end >= r.begin && r.end <= m.source.size()) edits.push_back({r.begin, r.end - r.begin, r.text});
  // an attribute insertion that falls inside a replaced span belongs to text that is going away
  edits.erase(std::remove_if(edits.begin(), edits.end(), [&](const Edit &e) {
                if (e.erase != 0) return false;
                for (const auto &r : m.replacements)
                  if (e.at > r.begin && e.at < r.end) return true;
                for (const auto &r : m.erasures)
                  if (e.at > r.first && e.at < r.second) return true;
                return false;
              }), edits.end());
  std::sort(edits.begin(), edits.end(), [](const Edit &a, const Edit &b) { return a.at > b.at; });
  std::string out = m.source;
  for (const Edit &e : edits) out.replace(e.at, e.erase, e.text);
  return out;
}

} // namespace front
} // namespace afir
