// TC language front-end: tree utilities, scanner, parser, semantic analysis, canonicalisation.
// Behaviour (token set, grammar, typing rules, error texts, printed trees) follows the reference's
// tc/lang so that the same TC text is accepted or rejected the same way and prints the same tree;
// the differential tests compare against the reference's own front-end.
#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <map>
#include <unordered_map>

#include "tc/lang/canonicalize.h"
#include "tc/lang/error_report.h"
#include "tc/lang/lexer.h"
#include "tc/lang/parser.h"
#include "tc/lang/sema.h"
#include "tc/lang/tree.h"

namespace lang {

// =============================================================================================
// kinds
// =============================================================================================
namespace {
struct KindEntry {
  int kind;
  const char* name;   // printed name
  const char* token;  // source spelling ("" = never produced by the scanner)
};
const KindEntry kKinds[] = {
    {TK_EOF, "eof", ""}, {TK_NUMBER, "number", ""}, {TK_BOOL_VALUE, "bool_value", ""},
    {TK_MIN, "min", "min"}, {TK_MAX, "max", "max"}, {TK_WHERE, "where", "where"},
    {TK_DEF, "def", "def"}, {TK_ARROW, "arrow", "->"}, {TK_EQUIVALENT, "equivalent", "<=>"},
    {TK_IDENT, "ident", ""}, {TK_STRING, "string", ""}, {TK_CONST, "const", ""},
    {TK_LIST, "list", ""}, {TK_OPTION, "option", ""}, {TK_APPLY, "apply", ""},
    {TK_COMPREHENSION, "comprehension", ""}, {TK_TENSOR_TYPE, "tensor_type", ""},
    {TK_RANGE_CONSTRAINT, "range_constraint", ""}, {TK_PARAM, "param", ""},
    {TK_INFERRED, "inferred", ""}, {TK_ACCESS, "access", ""}, {TK_BUILT_IN, "built-in", ""},
    {TK_PLUS_EQ, "plus_eq", "+="}, {TK_TIMES_EQ, "times_eq", "*="}, {TK_MIN_EQ, "min_eq", "min="},
    {TK_MAX_EQ, "max_eq", "max="}, {TK_PLUS_EQ_B, "plus_eq_b", "+=!"},
    {TK_TIMES_EQ_B, "times_eq_b", "*=!"}, {TK_MIN_EQ_B, "min_eq_b", "min=!"},
    {TK_MAX_EQ_B, "max_eq_b", "max=!"}, {TK_BOOL, "bool", "bool"}, {TK_UINT8, "uint8", "uint8"},
    {TK_UINT16, "uint16", "uint16"}, {TK_UINT32, "uint32", "uint32"}, {TK_UINT64, "uint64", "uint64"},
    {TK_INT8, "int8", "int8"}, {TK_INT16, "int16", "int16"}, {TK_INT32, "int32", "int32"},
    {TK_INT64, "int64", "int64"}, {TK_FLOAT16, "float16", "float16"},
    {TK_FLOAT32, "float32", "float32"}, {TK_FLOAT64, "float64", "float64"},
    {TK_FLOAT, "float", "float"}, {TK_DOUBLE, "double", "double"}, {TK_CAST, "cast", ""},
    {TK_IN, "in", "in"}, {TK_GE, "ge", ">="}, {TK_LE, "le", "<="}, {TK_EQ, "eq", "=="},
    {TK_NE, "neq", "!="}, {TK_AND, "and", "&&"}, {TK_OR, "or", "||"}, {TK_LET, "let", ""},
    {TK_EXISTS, "exists", "exists"},
};
const char kSingleCharTokens[] = "+-*/()[]?:,={}><!%";

const KindEntry* findKind(int kind) {
  for (const auto& e : kKinds)
    if (e.kind == kind) return &e;
  return nullptr;
}
}  // namespace

std::string kindToString(int kind) {
  if (kind < 256) return std::string(1, (char)kind);
  if (const KindEntry* e = findKind(kind)) return e->name;
  throw std::runtime_error("unknown kind: " + std::to_string(kind));
}

std::string kindToToken(int kind) {
  if (kind < 256) return std::string(1, (char)kind);
  const KindEntry* e = findKind(kind);
  if (!e) throw std::runtime_error("unknown kind: " + std::to_string(kind));
  if (!*e->token) throw std::runtime_error("No token for: " + kindToString(kind));
  return e->token;
}

bool isScalarTypeKind(int kind) { return kind >= TK_BOOL && kind <= TK_DOUBLE; }

// =============================================================================================
// source ranges and trees
// =============================================================================================
void SourceRange::highlight(std::ostream& out) const {
  const std::string& str = file();
  size_t lineBegin = start_, lineEnd = start_;
  while (lineBegin > 0 && str[lineBegin - 1] != '\n') --lineBegin;
  while (lineEnd < str.size() && str[lineEnd] != '\n') ++lineEnd;
  out << str.substr(0, lineEnd) << "\n";
  out << std::string(start_ - lineBegin, ' ');
  const size_t len = std::min(size(), lineEnd - start_);
  out << std::string(len, '~') << (len < size() ? "...  <--- HERE" : " <--- HERE");
  out << str.substr(lineEnd);
  if (!str.empty() && str.back() != '\n') out << "\n";
}

TreeRef Tree::number(double v) {
  auto t = std::make_shared<Tree>();
  t->kind_ = TK_NUMBER;
  t->payload_ = Payload::Number;
  t->number_ = v;
  return t;
}
TreeRef Tree::string(const std::string& s) {
  auto t = std::make_shared<Tree>();
  t->kind_ = TK_STRING;
  t->payload_ = Payload::String;
  t->string_ = s;
  return t;
}
TreeRef Tree::boolean(bool b) {
  auto t = std::make_shared<Tree>();
  t->kind_ = TK_BOOL_VALUE;
  t->payload_ = Payload::Bool;
  t->number_ = b ? 1 : 0;
  return t;
}
TreeRef Tree::compound(int kind, const SourceRange& range, TreeList trees) {
  auto t = std::make_shared<Tree>();
  t->kind_ = kind;
  size_t s = range.start(), e = range.end();
  for (const auto& c : trees) {
    if (c->isAtom()) continue;
    s = std::min(s, c->range().start());
    e = std::max(e, c->range().end());
  }
  t->range_.reset(new SourceRange(range.file_ptr(), s, e));
  t->trees_ = std::move(trees);
  return t;
}

TreeRef Tree::map(const std::function<TreeRef(TreeRef)>& fn) {
  if (isAtom()) return shared_from_this();
  TreeList mapped;
  mapped.reserve(trees_.size());
  for (const auto& c : trees_) mapped.push_back(fn(c));
  return compound(kind_, *range_, std::move(mapped));
}

void Tree::expect(int k, size_t numsubtrees) const {
  if (kind_ == k && trees_.size() == numsubtrees) return;
  std::stringstream ss;
  ss << "expected kind '" << kindToString(k) << "' with " << numsubtrees
     << " subtrees but found '" << kindToString(kind_) << "' with " << trees_.size()
     << " subtrees.\n";
  if (!isAtom()) range().highlight(ss);
  throw std::runtime_error(ss.str());
}

namespace {
constexpr size_t kPrintColumns = 40;

struct TreePrinter {
  std::unordered_map<const Tree*, std::string> flat;
  const std::string& flatten(const TreeRef& t) {
    auto it = flat.find(t.get());
    if (it != flat.end()) return it->second;
    std::stringstream out;
    if (t->kind() == TK_NUMBER) {
      out << t->doubleValue();
    } else if (t->kind() == TK_STRING) {
      out << t->stringValue();
    } else {
      out << "(" << kindToString(t->kind());
      for (const auto& c : t->trees()) out << " " << flatten(c);
      out << ")";
    }
    return flat.emplace(t.get(), out.str()).first->second;
  }
  void print(std::ostream& out, const TreeRef& t, size_t indent) {
    const std::string& s = flatten(t);
    if (indent + s.size() < kPrintColumns || t->isAtom()) {
      out << s;
      return;
    }
    out << "(" << kindToString(t->kind());
    for (const auto& c : t->trees()) {
      out << "\n" << std::string(indent + 2, ' ');
      print(out, c, indent + 2);
    }
    out << ")";
  }
};
}  // namespace

void printTree(std::ostream& out, const TreeRef& t) {
  TreePrinter p;
  p.print(out, t, 0);
  out << std::endl;
}
std::ostream& operator<<(std::ostream& out, const TreeRef& t) {
  printTree(out, t);
  return out;
}

// =============================================================================================
// scanner
// =============================================================================================
double Token::doubleValue() const { return std::strtod(text().c_str(), nullptr); }

int binaryPrecedence(int kind) {
  switch (kind) {
    case '?': return 1;
    case TK_OR: return 2;
    case TK_AND: return 3;
    case '>': case '<': case TK_LE: case TK_GE: case TK_EQ: case TK_NE: return 4;
    case '+': case '-': return 5;
    case '*': case '/': case '%': return 6;
    default: return 0;
  }
}
int unaryPrecedence(int kind) { return (kind == '-' || kind == '!') ? 7 : 0; }

Lexer::Lexer(const std::string& text)
    : file(std::make_shared<std::string>(text)), cur_(TK_EOF, SourceRange(file, 0, 0)) {
  next();
}

Token Lexer::next() {
  Token r = cur_;
  if (lookahead_) {
    cur_ = *lookahead_;
    lookahead_.reset();
  } else {
    cur_ = lex();
  }
  return r;
}
bool Lexer::nextIf(int kind) {
  if (cur_.kind != kind) return false;
  next();
  return true;
}
Token Lexer::lookahead() {
  if (!lookahead_) lookahead_.reset(new Token(lex()));
  return *lookahead_;
}
Token Lexer::expect(int kind) {
  if (cur_.kind != kind) reportError(kindToString(kind));
  return next();
}
void Lexer::reportError(const std::string& what) { reportError(what, cur_); }
void Lexer::reportError(const std::string& what, const Token& t) {
  throw ErrorReport(t.range) << "expected " << what << " but found '" << t.kindString()
                             << "' here:";
}

Token Lexer::lex() {
  const std::string& s = *file;
  size_t p = pos_;
  for (;;) {  // whitespace and comments
    while (p < s.size() && isspace((unsigned char)s[p])) ++p;
    if (p < s.size() && s[p] == '#') {
      while (p < s.size() && s[p] != '\n') ++p;
      continue;
    }
    break;
  }
  auto make = [&](int kind, size_t len) {
    pos_ = p + len;
    return Token(kind, SourceRange(file, p, p + len));
  };
  if (p == s.size()) return make(TK_EOF, 0);

  // numeric literal: what strtod takes, but never a leading sign ("1+3" is three tokens)
  if (s[p] != '-' && s[p] != '+') {
    const char* b = s.c_str() + p;
    char* e = nullptr;
    std::strtod(b, &e);
    if (e > b) return make(TK_NUMBER, (size_t)(e - b));
  }

  // longest match among identifiers and the fixed spellings
  size_t bestLen = 0;
  int bestKind = 0;
  size_t identLen = 0;
  while (p + identLen < s.size()) {
    const char c = s[p + identLen];
    if (isalpha((unsigned char)c) || c == '_' || (identLen > 0 && isdigit((unsigned char)c)))
      ++identLen;
    else
      break;
  }
  if (identLen) {
    bestLen = identLen;
    bestKind = TK_IDENT;
  }
  // a fixed spelling wins over an identifier of the same length ("max" is TK_MAX, "maxx" is not)
  for (const auto& e : kKinds) {
    const size_t n = strlen(e.token);
    if (n == 0 || s.compare(p, n, e.token) != 0) continue;
    if (n > bestLen || (n == bestLen && bestKind == TK_IDENT)) {
      bestLen = n;
      bestKind = e.kind;
    }
  }
  if (bestLen == 0 && strchr(kSingleCharTokens, s[p])) {
    bestLen = 1;
    bestKind = (unsigned char)s[p];
  }
  if (bestLen == 0)
    reportError("a valid token", Token((unsigned char)s[p], SourceRange(file, p, p + 1)));
  return make(bestKind, bestLen);
}

// =============================================================================================
// parser
// =============================================================================================
TreeRef Parser::parseIdent() {
  Token t = L.expect(TK_IDENT);
  return Ident::create(t.range, t.text());
}

TreeRef Parser::parseConst() {
  Token t = L.expect(TK_NUMBER);
  const std::string txt = t.text();
  // a literal is floating point iff it is spelled with '.' or an exponent
  const int type = (txt.find('.') != std::string::npos || txt.find('e') != std::string::npos)
                       ? TK_FLOAT : TK_INT32;
  return Const::create(t.range, Tree::number(t.doubleValue()), Tree::compound(type, t.range));
}

TreeRef Parser::parseScalarType() {
  if (!isScalarTypeKind(L.cur().kind)) L.reportError("a scalar type");
  Token t = L.next();
  return Tree::compound(t.kind, t.range);
}

TreeRef Parser::parseList(int begin, int sep, int end, const std::function<TreeRef()>& item) {
  SourceRange r = L.cur().range;
  L.expect(begin);
  TreeList elements;
  if (L.cur().kind != end) {
    do {
      elements.push_back(item());
    } while (L.nextIf(sep));
  }
  L.expect(end);
  return List::create(r, std::move(elements));
}

TreeRef Parser::parseBaseExp() {
  const int k = L.cur().kind;
  if (k == TK_NUMBER) return parseConst();
  if (k == '(') {
    L.next();
    TreeRef e = parseExp();
    L.expect(')');
    return e;
  }
  if (isScalarTypeKind(k)) {  // cast: float(expr)
    TreeRef type = parseScalarType();
    L.expect('(');
    TreeRef value = parseExp();
    L.expect(')');
    return Cast::create(type->range(), value, type);
  }
  if (k == TK_MIN || k == TK_MAX) {  // binary operators spelled as calls
    SourceRange r = L.cur().range;
    L.next();
    L.expect('(');
    TreeRef a = parseExp();
    L.expect(',');
    TreeRef b = parseExp();
    L.expect(')');
    return Tree::compound(k, r, {a, b});
  }
  TreeRef id = parseIdent();
  SourceRange r = L.cur().range;
  if (L.cur().kind == '(')
    return Apply::create(r, id, parseList('(', ',', ')', [&] { return parseExp(); }));
  if (L.nextIf('.')) {
    Token t = L.expect(TK_NUMBER);
    return Select::create(r, id, Tree::number(t.doubleValue()));
  }
  return id;
}

TreeRef Parser::parseExp(int precedence) {
  TreeRef lhs;
  if (int up = unaryPrecedence(L.cur().kind)) {
    const int kind = L.cur().kind;
    SourceRange r = L.cur().range;
    L.next();
    lhs = Tree::compound(kind, r, {parseExp(up)});
  } else {
    lhs = parseBaseExp();
  }
  for (;;) {
    int bp = binaryPrecedence(L.cur().kind);
    if (bp == 0 || bp <= precedence) break;
    const int kind = L.cur().kind;
    SourceRange r = L.cur().range;
    L.next();
    if (kind == '?') {  // right associative: a ? b : c ? d : e
      --bp;
      TreeRef yes = parseExp();
      L.expect(':');
      TreeRef no = parseExp(bp);
      lhs = Tree::compound('?', r, {lhs, yes, no});
      continue;
    }
    lhs = Tree::compound(kind, r, {lhs, parseExp(bp)});
  }
  return lhs;
}

TreeRef Parser::parseType() {
  TreeRef st = parseScalarType();
  TreeRef dims;
  if (L.cur().kind == '(') {
    dims = parseList('(', ',', ')', [&]() -> TreeRef {
      return L.cur().kind == TK_NUMBER ? parseConst() : parseIdent();
    });
  } else {
    dims = List::create(L.cur().range, {});
  }
  return TensorType::create(st->range(), st, dims);
}

TreeRef Parser::parseParam() {
  if (L.cur().kind == TK_IDENT) {
    TreeRef id = parseIdent();
    return Param::create(id->range(), id, Tree::compound(TK_INFERRED, id->range()));
  }
  TreeRef type = parseType();
  TreeRef id = parseIdent();
  return Param::create(type->range(), id, type);
}

TreeRef Parser::parseWhereClause() {
  const Token ahead = L.lookahead();
  if (ahead.kind == '=') {
    TreeRef id = parseIdent();
    L.expect('=');
    TreeRef e = parseExp();
    return Let::create(id->range(), id, e);
  }
  if (ahead.kind == TK_IN) {
    TreeRef id = parseIdent();
    L.expect(TK_IN);
    TreeRef lo = parseExp();
    L.expect(':');
    TreeRef hi = parseExp();
    return RangeConstraint::create(id->range(), id, lo, hi);
  }
  L.expect(TK_EXISTS);
  TreeRef e = parseExp();
  return Exists::create(e->range(), e);
}

TreeRef Parser::parseStmt() {
  TreeRef ident = parseIdent();
  TreeRef indices = L.cur().kind == '('
                        ? parseList('(', ',', ')', [&] { return parseIdent(); })
                        : List::create(L.cur().range, {});
  TreeRef assign;
  switch (L.cur().kind) {
    case TK_PLUS_EQ: case TK_TIMES_EQ: case TK_MIN_EQ: case TK_MAX_EQ:
    case TK_PLUS_EQ_B: case TK_TIMES_EQ_B: case TK_MIN_EQ_B: case TK_MAX_EQ_B: case '=': {
      const int kind = L.next().kind;
      assign = Tree::compound(kind, L.cur().range);
      break;
    }
    default:
      L.reportError("a valid assignment operator");
  }
  TreeRef rhs = parseExp();
  // optional "<=> name(accesses)"
  TreeRef equivalent;
  {
    SourceRange r = L.cur().range;
    if (L.nextIf(TK_EQUIVALENT)) {
      Token name = L.expect(TK_IDENT);
      TreeRef accesses = parseList('(', ',', ')', [&] { return parseExp(); });
      equivalent = Tree::compound(TK_OPTION, r, {Equivalent::create(r, name.text(), accesses)});
    } else {
      equivalent = Tree::compound(TK_OPTION, r);
    }
  }
  TreeRef where;
  if (L.nextIf(TK_WHERE)) {
    TreeList clauses;
    do {
      clauses.push_back(parseWhereClause());
    } while (L.nextIf(','));
    SourceRange r = clauses.at(0)->range();
    where = List::create(r, std::move(clauses));
  } else {
    where = List::create(L.cur().range, {});
  }
  TreeRef noReductionVars = Tree::compound(TK_LIST, ident->range());
  return Comprehension::create(ident->range(), ident, indices, assign, rhs, where, equivalent,
                               noReductionVars);
}

TreeRef Parser::parseFunction() {
  L.expect(TK_DEF);
  TreeRef name = parseIdent();
  TreeRef params = parseList('(', ',', ')', [&] { return parseParam(); });
  L.expect(TK_ARROW);
  TreeRef returns = parseList('(', ',', ')', [&] { return parseParam(); });
  L.expect('{');
  SourceRange r = L.cur().range;
  TreeList stmts;
  while (!L.nextIf('}')) stmts.push_back(parseStmt());
  return Def::create(name->range(), name, params, returns, List::create(r, std::move(stmts)));
}

// =============================================================================================
// semantic analysis
// =============================================================================================
TypeInfo::TypeInfo(const TreeRef& t) : code_(Int), bits_(0) {
  switch (t->kind()) {
    case TK_BOOL: code_ = UInt; bits_ = 1; break;
    case TK_UINT8: code_ = UInt; bits_ = 8; break;
    case TK_UINT16: code_ = UInt; bits_ = 16; break;
    case TK_UINT32: code_ = UInt; bits_ = 32; break;
    case TK_UINT64: code_ = UInt; bits_ = 64; break;
    case TK_INT8: code_ = Int; bits_ = 8; break;
    case TK_INT16: code_ = Int; bits_ = 16; break;
    case TK_INT32: code_ = Int; bits_ = 32; break;
    case TK_INT64: code_ = Int; bits_ = 64; break;
    case TK_FLOAT16: code_ = Float; bits_ = 16; break;
    case TK_FLOAT32: case TK_FLOAT: code_ = Float; bits_ = 32; break;
    case TK_FLOAT64: case TK_DOUBLE: code_ = Float; bits_ = 64; break;
    default:
      throw ErrorReport(t) << "Unhandled TC scalar type: " << t;
  }
  if (code_ == Float && bits_ == 16)
    throw ErrorReport(t) << "Half precision floating point not supported "
                         << "until we can make NVRTC include system headers";
}

int TypeInfo::toScalarToken() const {
  if (code_ == UInt) {
    switch (bits_) {
      case 1: return TK_BOOL;
      case 8: return TK_UINT8;
      case 16: return TK_UINT16;
      case 32: return TK_UINT32;
      case 64: return TK_UINT64;
    }
  } else if (code_ == Int) {
    switch (bits_) {
      case 8: return TK_INT8;
      case 16: return TK_INT16;
      case 32: return TK_INT32;
      case 64: return TK_INT64;
    }
  } else {
    switch (bits_) {
      case 16: return TK_FLOAT16;
      case 32: return TK_FLOAT;
      case 64: return TK_DOUBLE;
    }
  }
  throw std::runtime_error("Unknown type info?");
}

TreeRef match_types(const TreeRef& a, const TreeRef& b) {
  const TypeInfo ta(a), tb(b);
  if (ta == tb) return a;
  if (ta.is_float() != tb.is_float()) return ta.is_float() ? a : b;  // int op float -> float
  if (ta.is_float() || (ta.is_uint() && tb.is_uint())) return ta.bits() > tb.bits() ? a : b;
  // signed/unsigned integer mix: signed of the wider width
  return Tree::compound(TypeInfo(TypeInfo::Int, std::max(ta.bits(), tb.bits())).toScalarToken(),
                        a->range());
}

int builtinArity(const std::string& name) {
  static const std::unordered_map<std::string, int> table = {
      {"acos", 1}, {"acosh", 1}, {"asin", 1}, {"asinh", 1}, {"atan2", 2}, {"atan", 1},
      {"atanh", 1}, {"cbrt", 1}, {"ceil", 1}, {"copysign", 2}, {"cos", 1}, {"cosh", 1},
      {"cospi", 1}, {"cyl_bessel_i0", 1}, {"cyl_bessel_i1", 1}, {"erfc", 1}, {"erfcinv", 1},
      {"erfcx", 1}, {"erf", 1}, {"erfinv", 1}, {"exp10", 1}, {"exp2", 1}, {"exp", 1},
      {"expm1", 1}, {"fabs", 1}, {"fdim", 2}, {"fdivide", 2}, {"floor", 1}, {"fma", 3},
      {"fmax", 2}, {"fmin", 2}, {"fmod", 2}, {"hypot", 2}, {"j0", 1}, {"j1", 1}, {"lgamma", 1},
      {"log10", 1}, {"log1p", 1}, {"log2", 1}, {"logb", 1}, {"log", 1}, {"nextafter", 2},
      {"norm3d", 3}, {"norm4d", 4}, {"normcdf", 1}, {"normcdfinv", 1}, {"pow", 2}, {"rcbrt", 1},
      {"remainder", 2}, {"rhypot", 2}, {"rnorm3d", 3}, {"rnorm4d", 4}, {"round", 1}, {"rsqrt", 1},
      {"sin", 1}, {"sinh", 1}, {"sinpi", 1}, {"sqrt", 1}, {"tan", 1}, {"tanh", 1}, {"tgamma", 1},
      {"trunc", 1}, {"y0", 1}, {"y1", 1}};
  auto it = table.find(name);
  return it == table.end() ? -1 : it->second;
}

TreeRef Sema::typeOfExpr(const TreeRef& e) const {
  auto it = types_.find(e.get());
  if (it == types_.end())
    throw ErrorReport(e) << "INTERNAL ERROR: type not in map for expression " << e;
  return it->second;
}

TreeRef Sema::withType(const TreeRef& e, const TreeRef& type) {
  const bool inserted = types_.emplace(e.get(), type).second;
  TC_ASSERT(e, inserted);
  keepAlive_.push_back(e);
  return e;
}

TreeRef Sema::matchAllTypes(const TreeRef& list, TreeRef matched) {
  for (const auto& e : list->trees())
    matched = matched ? match_types(matched, typeOfExpr(e)) : typeOfExpr(e);
  return matched;
}

TreeRef Sema::expectIntegral(const TreeRef& e) {
  if (TypeInfo(typeOfExpr(e)).code() == TypeInfo::Float)
    throw ErrorReport(e) << " expected integral type but found "
                         << kindToString(typeOfExpr(e)->kind());
  return e;
}

void Sema::insert(Env& env, const Ident& id, const TreeRef& value, bool mustBeUndefined) {
  const std::string& name = id.name();
  if (builtinArity(name) >= 0)
    throw ErrorReport(id) << "'" << name << "' is a built-in function and cannot be redefined";
  const bool fresh = env.emplace(name, value).second;
  if (mustBeUndefined && !fresh) throw ErrorReport(id) << name << " already defined";
}

TreeRef Sema::lookupIn(Env& env, const Ident& id, bool required) {
  auto it = env.find(id.name());
  if (it == env.end()) {
    if (required) throw ErrorReport(id) << "undefined variable " << id.name() << " used here.";
    return nullptr;
  }
  return it->second;
}

TreeRef Sema::lookup(const Ident& id, bool required) {
  if (TreeRef v = lookupIn(indexEnv_, id, false)) return v;
  if (TreeRef v = lookupIn(letEnv_, id, false)) return v;
  return lookupIn(env_, id, required);
}

TreeRef Sema::lookupVarOrCreateIndex(const Ident& id) {
  TreeRef type = lookup(id, false);
  if (!type) {  // first use of an unknown name on the right-hand side: a reduction index
    type = scalar(TK_INT32, id);
    insert(indexEnv_, id, type, true);
    reductionVars_.push_back(id);
  }
  return type;
}

TreeRef Sema::checkExp(const TreeRef& e, bool allowAccess) {
  auto recurse = [&](const TreeRef& t) {
    return t->map([&](TreeRef c) { return checkExp(c, allowAccess); });
  };
  switch (e->kind()) {
    case TK_APPLY: {
      Apply a(e);
      if (!allowAccess) throw ErrorReport(e) << "tensor accesses cannot be used in this context";
      Ident id = a.name();
      const int arity = builtinArity(id.name());
      if (arity >= 0) {
        if ((size_t)arity != a.arguments().size())
          throw ErrorReport(e) << "expected " << arity << " but found " << a.arguments().size();
        TreeRef args = checkExp(a.arguments(), allowAccess);
        // built-ins compute in floating point: an integer literal argument is promoted
        TreeRef type = matchAllTypes(args, scalar(TK_FLOAT, e));
        return withType(BuiltIn::create(e->range(), id.name(), args, type), type);
      }
      TreeRef t = lookup(id, true);
      if (t->kind() != TK_TENSOR_TYPE)
        throw ErrorReport(id) << "expected a tensor but found a scalar";
      TensorType tt(t);
      if (tt.dims().size() != a.arguments().size())
        throw ErrorReport(a) << "expected " << tt.dims().size() << " dimensions but found "
                             << a.arguments().size() << " dimensions.";
      TreeRef checked = checkExp(a.arguments(), allowAccess);
      for (const auto& idx : checked->trees()) expectIntegral(idx);
      return withType(Access::create(e->range(), id, checked), tt.scalarTypeTree());
    }
    case TK_IDENT: {
      Ident id(e);
      TreeRef type = lookupVarOrCreateIndex(id);
      if (type->kind() == TK_TENSOR_TYPE) {
        if (TensorType(type).dims().size() != 0)
          throw ErrorReport(e) << "expected a scalar but found a tensor expression.";
        // a 0-dimensional tensor used by name is an access with no indices
        return checkExp(Apply::create(id.range(), id, List::create(id.range(), {})), allowAccess);
      }
      return withType(e, type);
    }
    case '.': {
      Select s(e);
      TreeRef t = lookup(s.name(), true);
      if (t->kind() != TK_TENSOR_TYPE)
        throw ErrorReport(s.name()) << "expected a tensor but found a scalar";
      return withType(e, scalar(TK_INT32, e));
    }
    case '+': case '-': case '*': case '/': case '%': case TK_MIN: case TK_MAX: {
      TreeRef n = recurse(e);
      return withType(n, matchAllTypes(n));
    }
    case TK_EQ: case TK_NE: case TK_GE: case TK_LE: case '<': case '>': {
      TreeRef n = recurse(e);
      matchAllTypes(n);
      return withType(n, scalar(TK_BOOL, e));
    }
    case TK_AND: case TK_OR: case '!': {
      TreeRef n = recurse(e);
      const int k = matchAllTypes(n)->kind();
      if (k != TK_BOOL) throw ErrorReport(e) << "expected boolean but found " << kindToString(k);
      return withType(n, scalar(TK_BOOL, e));
    }
    case '?': {
      TreeRef n = recurse(e);
      const int k = typeOfExpr(n->tree(0))->kind();
      if (k != TK_BOOL)
        throw ErrorReport(n->tree(0)) << "expected boolean but found " << kindToString(k);
      return withType(n, match_types(typeOfExpr(n->tree(1)), typeOfExpr(n->tree(2))));
    }
    case TK_CONST:
      return withType(e, Const(e).type());
    case TK_CAST: {
      Cast c(e);
      TreeRef v = checkExp(c.value(), allowAccess);
      match_types(typeOfExpr(v), c.type());
      return withType(Cast::create(c.range(), v, c.type()), c.type());
    }
    case TK_LIST:
      return recurse(e);
    default:
      throw ErrorReport(e) << "NYI - semantic checking for " << e;
  }
}

TreeRef Sema::checkParam(const TreeRef& param) {
  Param p(param);
  TensorType tt(p.type());
  for (const auto& d : tt.dims())
    if (d->kind() == TK_IDENT) insert(env_, Ident(d), scalar(TK_INT32, d), false);
  insert(env_, p.ident(), p.type(), true);
  return param;
}

TreeRef Sema::checkWhereClause(const TreeRef& clause) {
  if (clause->kind() == TK_LET) {
    Let l(clause);
    TreeRef rhs = checkExp(l.rhs(), true);
    insert(letEnv_, l.name(), typeOfExpr(rhs), true);
    return Let::create(l.range(), l.name(), rhs);
  }
  if (clause->kind() == TK_EXISTS)
    return Exists::create(clause->range(), checkExp(Exists(clause).exp(), true));
  RangeConstraint rc(clause);
  lookupVarOrCreateIndex(rc.ident());
  lookupIn(indexEnv_, rc.ident(), true);
  TreeRef lo = expectIntegral(checkExp(rc.start(), false));
  TreeRef hi = expectIntegral(checkExp(rc.end(), false));
  return RangeConstraint::create(rc.range(), rc.ident(), lo, hi);
}

TreeRef Sema::checkStmt(const TreeRef& stmtTree) {
  Comprehension stmt(stmtTree);
  for (const auto& idx : stmt.indices()) insert(indexEnv_, idx, scalar(TK_INT32, idx), true);

  const std::string name = stmt.ident().name();
  if (inputs_.count(name)) throw ErrorReport(stmtTree) << "TC inputs are immutable";

  // the output's dimensions get the symbolic names <tensor>.<k>
  TreeList outputDims;
  const int rank = (int)stmt.indices().size();
  for (int i = 0; i < rank; ++i)
    outputDims.push_back(Ident::create(stmt.range(), name + "." + std::to_string(i)));

  TreeRef where = stmt.whereClauses().map([&](const TreeRef& c) { return checkWhereClause(c); });
  TreeRef rhs = checkExp(stmt.rhs(), true);
  TreeRef scalarType = typeOfExpr(rhs);

  auto annotated = annotatedOutputs_.find(name);
  if (annotated != annotatedOutputs_.end()) {
    TensorType tt(annotated->second);
    TreeRef matched = match_types(scalarType, tt.scalarTypeTree());
    if (tt.scalarTypeTree()->kind() != matched->kind())
      throw ErrorReport(stmt) << " attempting to assign type " << kindToString(scalarType->kind())
                              << " to narrower type " << kindToString(tt.scalarTypeTree()->kind())
                              << " without an explicit cast";
    if (tt.dims().size() != stmt.indices().size())
      throw ErrorReport(stmt) << " tensor defined with " << stmt.indices().size()
                              << " dimensions but declared as an output with " << tt.dims().size()
                              << " dimensions.";
  }

  const int assign = stmt.assignment()->kind();
  const bool plainReduction =
      assign == TK_PLUS_EQ || assign == TK_TIMES_EQ || assign == TK_MIN_EQ || assign == TK_MAX_EQ;
  if (plainReduction && !lookup(stmt.ident(), false)) {
    ErrorReport err(stmt);
    const std::string tk = kindToToken(assign);
    err << "Reduction without initialization. If " << name
        << " is not pre-initialized before calling the TC function,"
        << " consider using the !-suffixed reduction operator " << tk << "! instead of " << tk;
    warn(err, opts_);
  }

  insert(env_, stmt.ident(),
         TensorType::create(stmt.range(), scalarType, List::create(stmt.range(), std::move(outputDims))),
         false);

  TreeRef equivalent = stmt.equivalentOption()->map([&](TreeRef eqTree) {
    Equivalent eq(eqTree);
    TreeRef accesses = eq.accesses().map([&](const TreeRef& a) { return checkExp(a, true); });
    return Equivalent::create(eq.range(), eq.name(), accesses);
  });

  if (!reductionVars_.empty() && assign == '=')
    throw ErrorReport(stmt) << "this statement includes reduction variable '"
                            << Ident(reductionVars_.back()).name()
                            << "' but does not specify a reduction.";

  TreeRef reductionList = List::create(stmt.ident().range(), std::move(reductionVars_));
  reductionVars_.clear();
  TreeRef result = Comprehension::create(stmt.range(), stmt.ident(), stmt.indices(),
                                         stmt.assignment(), rhs, where, equivalent, reductionList);
  if (!nonTemporaries_.count(name))
    throw ErrorReport(stmt) << name
                            << " is not listed as an input or output to this function. "
                               "Temporaries tensors are not yet implemented";
  indexEnv_.clear();
  letEnv_.clear();
  return result;
}

TreeRef Sema::checkFunction(const TreeRef& defTree) {
  Def def(defTree);
  auto mapList = [](const TreeRef& list, const std::function<TreeRef(TreeRef)>& fn) {
    TreeList out;
    for (const auto& e : list->trees()) out.push_back(fn(e));
    return List::create(list->range(), std::move(out));
  };
  TreeRef params = mapList(def.params(), [&](TreeRef p) { return checkParam(p); });
  for (const auto& r : def.returns())
    if (!r.typeIsInferred()) annotatedOutputs_.emplace(r.ident().name(), r.tensorType());
  for (const auto& p : def.params()) {
    nonTemporaries_.insert(p.ident().name());
    inputs_.insert(p.ident().name());
  }
  for (const auto& r : def.returns()) nonTemporaries_.insert(r.ident().name());
  TreeRef stmts = mapList(def.statements(), [&](TreeRef s) { return checkStmt(s); });
  TreeRef returns = mapList(def.returns(), [&](TreeRef r) {
    lookupIn(env_, Param(r).ident(), true);  // every declared output must have been written
    return r;
  });
  return Def::create(def.range(), def.name(), params, returns, stmts);
}

std::string Sema::dumpEnv() const {
  std::map<std::string, TreeRef> sorted(env_.begin(), env_.end());
  std::stringstream ss;
  for (const auto& kv : sorted) ss << kv.first << ": " << kv.second;
  return ss.str();
}

// =============================================================================================
// canonicalisation
// =============================================================================================
TreeRef canonicalize(const TreeRef& checkedDef) {
  std::unordered_map<std::string, std::string> names;
  std::function<TreeRef(TreeRef)> apply = [&](TreeRef n) -> TreeRef {
    if (n->kind() == TK_IDENT) {
      const std::string& old = Ident(n).name();
      auto it = names.find(old);
      if (it == names.end()) it = names.emplace(old, "i" + std::to_string(names.size())).first;
      return Ident::create(n->range(), it->second);
    }
    if (n->kind() == TK_APPLY)
      throw ErrorReport(n) << "canonicalize is only valid on trees after Sema has been run "
                           << "but it encountered a TK_APPLY node, which Sema removes";
    return n->map(apply);
  };
  return apply(checkedDef);
}

CanonicalTcString canonicalTc(const TreeRef& parsedDef) {
  std::stringstream ss;
  ss << canonicalize(Sema().checkFunction(parsedDef));
  return CanonicalTcString(ss.str());
}
CanonicalTcString canonicalTc(const std::string& tc) {
  return canonicalTc(Parser(tc).parseFunction());
}

}  // namespace lang
