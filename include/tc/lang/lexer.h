// Scanner for the TC language: whitespace and '#' comments are skipped; a numeric literal is
// whatever strtod accepts without a leading sign; identifiers are [A-Za-z_][A-Za-z0-9_]*;
// keywords, type names and multi-character operators win over identifiers only when they are the
// longest match (so "min_x" is an identifier and "min=!" one token).  Token set and precedences
// follow tc/lang/lexer.h:37-92,138-148 of the reference.
#pragma once

#include <memory>
#include <string>

#include "tc/lang/error_report.h"
#include "tc/lang/tree.h"

namespace lang {

struct Token {
  int kind;
  SourceRange range;
  Token(int k, const SourceRange& r) : kind(k), range(r) {}
  std::string text() const { return range.text(); }
  double doubleValue() const;
  std::string kindString() const { return kindToString(kind); }
};

// Operator precedence (0 = not an operator).  Binary, low to high: ?:, ||, &&, comparisons, + -,
// * / %.  Unary - and ! bind tighter than every binary operator.
int binaryPrecedence(int kind);
int unaryPrecedence(int kind);

class Lexer {
 public:
  explicit Lexer(const std::string& text);
  Token& cur() { return cur_; }
  Token next();                 // returns the current token and advances
  bool nextIf(int kind);        // advances iff the current token has this kind
  Token lookahead();            // the token after the current one
  Token expect(int kind);       // next() or "expected <kind> but found '<kind>' here:"
  [[noreturn]] void reportError(const std::string& what);
  [[noreturn]] void reportError(const std::string& what, const Token& t);
  std::shared_ptr<std::string> file;

 private:
  Token lex();
  size_t pos_ = 0;
  Token cur_;
  std::unique_ptr<Token> lookahead_;
};

}  // namespace lang
