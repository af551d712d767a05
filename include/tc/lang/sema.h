// Semantic analysis of a parsed def (the reference's tc/lang/sema.h:173-720):
//   * every expression gets a scalar type; arithmetic promotes int -> float and to the wider width;
//   * identifiers that are not tensors, sizes or let-bindings are index variables; those that do
//     not appear on the left-hand side are reduction variables, in order of first use, and are
//     recorded in the comprehension's last child;
//   * Apply nodes become Access (tensor read) or BuiltIn (math function) nodes;
//   * inputs are immutable, every written tensor must be a declared output, a reduction variable
//     needs a reduction operator, "+=!" without reduction variables degrades to "=".
#pragma once

#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "tc/lang/error_report.h"
#include "tc/lang/tree.h"
#include "tc/utils/compiler_options.h"

namespace lang {

// Scalar type algebra.
struct TypeInfo {
  enum Code { Int, UInt, Float };
  TypeInfo(Code c, int bits) : code_(c), bits_(bits) {}
  explicit TypeInfo(const TreeRef& scalarType);
  int toScalarToken() const;
  Code code() const { return code_; }
  int bits() const { return bits_; }
  bool is_float() const { return code_ == Float; }
  bool is_uint() const { return code_ == UInt; }
  bool operator==(const TypeInfo& o) const { return code_ == o.code_ && bits_ == o.bits_; }

 private:
  Code code_;
  int bits_;
};
TreeRef match_types(const TreeRef& a, const TreeRef& b);

// Number of arguments of a built-in math function, or -1 if `name` is not one.
int builtinArity(const std::string& name);

class Sema {
 public:
  explicit Sema(const tc::CompilerOptions& opts = tc::CompilerOptions()) : opts_(opts) {}
  TreeRef checkFunction(const TreeRef& def);
  TreeRef typeOfExpr(const TreeRef& e) const;
  // "name: <type tree>" for every tensor and size symbol, sorted by name.
  std::string dumpEnv() const;

 private:
  using Env = std::unordered_map<std::string, TreeRef>;
  TreeRef checkExp(const TreeRef& e, bool allowAccess);
  TreeRef checkStmt(const TreeRef& stmt);
  TreeRef checkParam(const TreeRef& param);
  TreeRef checkWhereClause(const TreeRef& clause);
  TreeRef withType(const TreeRef& e, const TreeRef& type);
  TreeRef matchAllTypes(const TreeRef& list, TreeRef matched = nullptr);
  TreeRef expectIntegral(const TreeRef& e);
  TreeRef lookupVarOrCreateIndex(const Ident& id);
  TreeRef lookup(const Ident& id, bool required);
  TreeRef lookupIn(Env& env, const Ident& id, bool required);
  void insert(Env& env, const Ident& id, const TreeRef& value, bool mustBeUndefined);
  TreeRef scalar(int kind, const TreeRef& anchor) { return Tree::compound(kind, anchor->range()); }

  std::vector<TreeRef> reductionVars_;  // per statement, first-use order
  Env indexEnv_, letEnv_;               // per statement
  Env env_;                             // tensors and size symbols
  Env annotatedOutputs_;
  std::unordered_map<const Tree*, TreeRef> types_;
  std::vector<TreeRef> keepAlive_;      // keeps typed expression nodes (and their addresses) alive
  std::unordered_set<std::string> inputs_, nonTemporaries_;
  tc::CompilerOptions opts_;
};

}  // namespace lang
