// Recursive-descent / precedence-climbing parser for TC (grammar: docs/source/semantics.rst and
// tc/lang/parser.h:23-317 of the reference):
//   def name(type(dims) id, ...) -> (id | type(dims) id, ...) { stmt* }
//   stmt: id(idx,...) (=|+=|*=|min=|max=|+=!|*=!|min=!|max=!) expr [<=> name(args)] [where clause,...]
//   clause: id in expr:expr | id = expr | exists expr
#pragma once

#include <functional>
#include <string>

#include "tc/lang/lexer.h"

namespace lang {

class Parser {
 public:
  explicit Parser(const std::string& text) : L(text) {}
  TreeRef parseFunction();
  TreeRef parseStmt();
  TreeRef parseExp(int precedence = 0);
  TreeRef parseIdent();
  TreeRef parseConst();
  TreeRef parseType();
  TreeRef parseParam();
  Lexer L;

 private:
  TreeRef parseBaseExp();
  TreeRef parseScalarType();
  TreeRef parseList(int begin, int sep, int end, const std::function<TreeRef()>& item);
  TreeRef parseWhereClause();
};

}  // namespace lang
