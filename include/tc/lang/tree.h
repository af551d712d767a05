// AST of the Tensor Comprehensions language.
//
// One node type (Tree) with a kind tag, a source range, an optional payload (number or string)
// and children; thin typed views (Def, Param, Comprehension, ...) name the children.  Kinds, view
// names and the s-expression printer follow the reference's tc/lang (token table
// tc/lang/lexer.h:37-92, views tc/lang/tree_views.h:34-99,357-439, printer tc/lang/tree.h:175-230)
// so trees print identically and the reference's call sites (lang::Def(t).name().name(), ...)
// read the same.
#pragma once

#include <functional>
#include <memory>
#include <ostream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace lang {

// Single characters are their own kind; named kinds start above the char range.
enum TokenKind : int {
  TK_DUMMY_START = 256,
  TK_EOF, TK_NUMBER, TK_BOOL_VALUE, TK_MIN, TK_MAX, TK_WHERE, TK_DEF, TK_ARROW, TK_EQUIVALENT,
  TK_IDENT, TK_STRING, TK_CONST, TK_LIST, TK_OPTION, TK_APPLY, TK_COMPREHENSION, TK_TENSOR_TYPE,
  TK_RANGE_CONSTRAINT, TK_PARAM, TK_INFERRED, TK_ACCESS, TK_BUILT_IN,
  TK_PLUS_EQ, TK_TIMES_EQ, TK_MIN_EQ, TK_MAX_EQ, TK_PLUS_EQ_B, TK_TIMES_EQ_B, TK_MIN_EQ_B, TK_MAX_EQ_B,
  TK_BOOL, TK_UINT8, TK_UINT16, TK_UINT32, TK_UINT64, TK_INT8, TK_INT16, TK_INT32, TK_INT64,
  TK_FLOAT16, TK_FLOAT32, TK_FLOAT64, TK_FLOAT, TK_DOUBLE,
  TK_CAST, TK_IN, TK_GE, TK_LE, TK_EQ, TK_NE, TK_AND, TK_OR, TK_LET, TK_EXISTS,
};

// Printable name of a kind ("plus_eq_b", "ident", "+") and the spelling the lexer matches for it.
std::string kindToString(int kind);
std::string kindToToken(int kind);
bool isScalarTypeKind(int kind);

// A span of the shared source text, with caret-style highlighting for error messages.
class SourceRange {
 public:
  SourceRange(std::shared_ptr<std::string> file, size_t start, size_t end)
      : file_(std::move(file)), start_(start), end_(end) {}
  std::string text() const { return file_->substr(start_, end_ - start_); }
  size_t size() const { return end_ - start_; }
  size_t start() const { return start_; }
  size_t end() const { return end_; }
  const std::string& file() const { return *file_; }
  const std::shared_ptr<std::string>& file_ptr() const { return file_; }
  void highlight(std::ostream& out) const;

 private:
  std::shared_ptr<std::string> file_;
  size_t start_, end_;
};

struct Tree;
using TreeRef = std::shared_ptr<Tree>;
using TreeList = std::vector<TreeRef>;

struct Tree : std::enable_shared_from_this<Tree> {
  enum class Payload { None, Number, String, Bool };

  int kind() const { return kind_; }
  bool isAtom() const { return payload_ != Payload::None; }
  const SourceRange& range() const {
    if (isAtom()) throw std::runtime_error("is an Atom");
    return *range_;
  }
  double doubleValue() const {
    if (payload_ != Payload::Number) throw std::runtime_error("not a TK_NUMBER");
    return number_;
  }
  const std::string& stringValue() const {
    if (payload_ != Payload::String) throw std::runtime_error("not a TK_STRING");
    return string_;
  }
  bool boolValue() const {
    if (payload_ != Payload::Bool) throw std::runtime_error("not a TK_BOOL_VALUE");
    return number_ != 0;
  }
  const TreeList& trees() const { return trees_; }
  const TreeRef& tree(size_t i) const { return trees_.at(i); }
  // New compound node of the same kind/range whose children are fn(child); atoms map to themselves.
  TreeRef map(const std::function<TreeRef(TreeRef)>& fn);
  void expect(int k) const { expect(k, trees_.size()); }
  void expect(int k, size_t numsubtrees) const;

  static TreeRef number(double v);
  static TreeRef string(const std::string& s);
  static TreeRef boolean(bool b);
  // The range of a compound grows to cover its (non-atom) children.
  static TreeRef compound(int kind, const SourceRange& range, TreeList trees = {});

 private:
  int kind_ = 0;
  Payload payload_ = Payload::None;
  double number_ = 0;
  std::string string_;
  std::unique_ptr<SourceRange> range_;
  TreeList trees_;
};

// Factories under the reference's names (String::create, Number::create, Compound::create).
struct String { static TreeRef create(const std::string& s) { return Tree::string(s); } };
struct Number { static TreeRef create(double v) { return Tree::number(v); } };
struct Bool { static TreeRef create(bool b) { return Tree::boolean(b); } };
struct Compound {
  static TreeRef create(int kind, const SourceRange& r, TreeList trees = {}) {
    return Tree::compound(kind, r, std::move(trees));
  }
};

// S-expression printer: a subtree is printed flat when it fits in 40 columns at its indent,
// otherwise one child per line indented by two.  Always ends with a newline.
void printTree(std::ostream& out, const TreeRef& t);
std::ostream& operator<<(std::ostream& out, const TreeRef& t);

// ---------------------------------------------------------------------------------------------
// Typed views
// ---------------------------------------------------------------------------------------------
struct TreeView {
  explicit TreeView(const TreeRef& t) : tree_(t) {}
  TreeRef tree() const { return tree_; }
  const SourceRange& range() const { return tree_->range(); }
  operator TreeRef() const { return tree_; }

 protected:
  TreeRef subtree(size_t i) const { return tree_->tree(i); }
  TreeRef tree_;
};

template <typename T>
struct ListView : TreeView {
  explicit ListView(const TreeRef& t) : TreeView(t) { t->expect(TK_LIST); }
  struct iterator {
    TreeList::const_iterator it;
    bool operator!=(const iterator& o) const { return it != o.it; }
    T operator*() const { return T(*it); }
    void operator++() { ++it; }
  };
  iterator begin() const { return iterator{tree_->trees().begin()}; }
  iterator end() const { return iterator{tree_->trees().end()}; }
  T operator[](size_t i) const { return T(tree_->trees().at(i)); }
  size_t size() const { return tree_->trees().size(); }
  bool empty() const { return size() == 0; }
  TreeRef map(const std::function<TreeRef(const T&)>& fn) const {
    return tree_->map([&](TreeRef v) { return fn(T(v)); });
  }
  static TreeRef create(const SourceRange& r, TreeList elements) {
    return Tree::compound(TK_LIST, r, std::move(elements));
  }
};
using List = ListView<TreeRef>;

struct Ident : TreeView {
  explicit Ident(const TreeRef& t) : TreeView(t) { t->expect(TK_IDENT, 1); }
  const std::string& name() const { return subtree(0)->stringValue(); }
  static TreeRef create(const SourceRange& r, const std::string& name) {
    return Tree::compound(TK_IDENT, r, {Tree::string(name)});
  }
};

template <int K>
struct ApplyLike : TreeView {
  explicit ApplyLike(const TreeRef& t) : TreeView(t) { t->expect(K, 2); }
  Ident name() const { return Ident(subtree(0)); }
  List arguments() const { return List(subtree(1)); }
  static TreeRef create(const SourceRange& r, TreeRef name, TreeRef args) {
    return Tree::compound(K, r, {name, args});
  }
};
using Apply = ApplyLike<TK_APPLY>;    // before Sema: tensor access or builtin call
using Access = ApplyLike<TK_ACCESS>;  // after Sema: tensor access

struct BuiltIn : TreeView {
  explicit BuiltIn(const TreeRef& t) : TreeView(t) { t->expect(TK_BUILT_IN, 3); }
  const std::string& name() const { return subtree(0)->stringValue(); }
  List arguments() const { return List(subtree(1)); }
  TreeRef type() const { return subtree(2); }
  static TreeRef create(const SourceRange& r, const std::string& name, TreeRef args, TreeRef type) {
    return Tree::compound(TK_BUILT_IN, r, {Tree::string(name), args, type});
  }
};

struct TensorType : TreeView {
  explicit TensorType(const TreeRef& t) : TreeView(t) { t->expect(TK_TENSOR_TYPE, 2); }
  TreeRef scalarTypeTree() const { return subtree(0); }
  int scalarType() const { return subtree(0)->kind(); }
  List dims() const { return List(subtree(1)); }
  static TreeRef create(const SourceRange& r, TreeRef scalar, TreeRef dims) {
    return Tree::compound(TK_TENSOR_TYPE, r, {scalar, dims});
  }
};

struct Param : TreeView {
  explicit Param(const TreeRef& t) : TreeView(t) { t->expect(TK_PARAM, 2); }
  Ident ident() const { return Ident(subtree(0)); }
  TreeRef type() const { return subtree(1); }
  bool typeIsInferred() const { return type()->kind() == TK_INFERRED; }
  TensorType tensorType() const { return TensorType(type()); }
  static TreeRef create(const SourceRange& r, TreeRef ident, TreeRef type) {
    return Tree::compound(TK_PARAM, r, {ident, type});
  }
};

struct Equivalent : TreeView {
  explicit Equivalent(const TreeRef& t) : TreeView(t) { t->expect(TK_EQUIVALENT, 2); }
  const std::string& name() const { return subtree(0)->stringValue(); }
  List accesses() const { return List(subtree(1)); }
  static TreeRef create(const SourceRange& r, const std::string& name, TreeRef accesses) {
    return Tree::compound(TK_EQUIVALENT, r, {Tree::string(name), accesses});
  }
};

struct RangeConstraint : TreeView {
  explicit RangeConstraint(const TreeRef& t) : TreeView(t) { t->expect(TK_RANGE_CONSTRAINT, 3); }
  Ident ident() const { return Ident(subtree(0)); }
  TreeRef start() const { return subtree(1); }
  TreeRef end() const { return subtree(2); }
  static TreeRef create(const SourceRange& r, TreeRef ident, TreeRef start, TreeRef end) {
    return Tree::compound(TK_RANGE_CONSTRAINT, r, {ident, start, end});
  }
};

struct Let : TreeView {
  explicit Let(const TreeRef& t) : TreeView(t) { t->expect(TK_LET, 2); }
  Ident name() const { return Ident(subtree(0)); }
  TreeRef rhs() const { return subtree(1); }
  static TreeRef create(const SourceRange& r, TreeRef name, TreeRef rhs) {
    return Tree::compound(TK_LET, r, {name, rhs});
  }
};

struct Exists : TreeView {
  explicit Exists(const TreeRef& t) : TreeView(t) { t->expect(TK_EXISTS, 1); }
  TreeRef exp() const { return subtree(0); }
  static TreeRef create(const SourceRange& r, TreeRef exp) {
    return Tree::compound(TK_EXISTS, r, {exp});
  }
};

struct Const : TreeView {
  explicit Const(const TreeRef& t) : TreeView(t) { t->expect(TK_CONST, 2); }
  double value() const { return subtree(0)->doubleValue(); }
  TreeRef type() const { return subtree(1); }
  static TreeRef create(const SourceRange& r, TreeRef value, TreeRef type) {
    return Tree::compound(TK_CONST, r, {value, type});
  }
};

struct Cast : TreeView {
  explicit Cast(const TreeRef& t) : TreeView(t) { t->expect(TK_CAST, 2); }
  TreeRef value() const { return subtree(0); }
  TreeRef type() const { return subtree(1); }
  static TreeRef create(const SourceRange& r, TreeRef value, TreeRef type) {
    return Tree::compound(TK_CAST, r, {value, type});
  }
};

struct Select : TreeView {  // T.k : size of dimension k of tensor T
  explicit Select(const TreeRef& t) : TreeView(t) { t->expect('.', 2); }
  Ident name() const { return Ident(subtree(0)); }
  int index() const { return (int)subtree(1)->doubleValue(); }
  static TreeRef create(const SourceRange& r, TreeRef name, TreeRef index) {
    return Tree::compound('.', r, {name, index});
  }
};

struct Comprehension : TreeView {
  explicit Comprehension(const TreeRef& t) : TreeView(t) { t->expect(TK_COMPREHENSION, 7); }
  Ident ident() const { return Ident(subtree(0)); }
  ListView<Ident> indices() const { return ListView<Ident>(subtree(1)); }
  TreeRef assignment() const { return subtree(2); }
  TreeRef rhs() const { return subtree(3); }
  List whereClauses() const { return List(subtree(4)); }
  TreeRef equivalentOption() const { return subtree(5); }
  ListView<Ident> reductionVariables() const { return ListView<Ident>(subtree(6)); }
  static TreeRef create(const SourceRange& r, TreeRef ident, TreeRef indices, TreeRef assignment,
                        TreeRef rhs, TreeRef where, TreeRef equivalent, TreeRef reductionVars) {
    return Tree::compound(TK_COMPREHENSION, r,
                          {ident, indices, assignment, rhs, where, equivalent, reductionVars});
  }
};

struct Def : TreeView {
  explicit Def(const TreeRef& t) : TreeView(t) { t->expect(TK_DEF, 4); }
  Ident name() const { return Ident(subtree(0)); }
  ListView<Param> params() const { return ListView<Param>(subtree(1)); }
  ListView<Param> returns() const { return ListView<Param>(subtree(2)); }
  ListView<Comprehension> statements() const { return ListView<Comprehension>(subtree(3)); }
  static TreeRef create(const SourceRange& r, TreeRef name, TreeRef params, TreeRef returns,
                        TreeRef stmts) {
    return Tree::compound(TK_DEF, r, {name, params, returns, stmts});
  }
};

}  // namespace lang
