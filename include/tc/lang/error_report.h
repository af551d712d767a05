// lang::ErrorReport — the exception every front-end / shape / matching error is reported with.
// what() is "\n<message>:\n<source with the offending span underlined>" like the reference's
// (tc/lang/error_report.h:23-64); tests match substrings of it.
#pragma once

#include <exception>
#include <iostream>
#include <sstream>
#include <string>

#include "tc/lang/tree.h"
#include "tc/utils/compiler_options.h"

namespace lang {

class ErrorReport : public std::exception {
 public:
  explicit ErrorReport(const TreeRef& context) : context_(context->range()) {}
  explicit ErrorReport(SourceRange range) : context_(std::move(range)) {}
  ErrorReport(const ErrorReport& e) : msg_(e.msg_.str()), context_(e.context_) {}

  const char* what() const noexcept override {
    std::stringstream out;
    out << "\n" << msg_.str() << ":\n";
    context_.highlight(out);
    rendered_ = out.str();
    return rendered_.c_str();
  }

  template <typename T>
  const ErrorReport& operator<<(const T& t) const {
    msg_ << t;
    return *this;
  }

 private:
  mutable std::stringstream msg_;
  SourceRange context_;
  mutable std::string rendered_;
};

inline void warn(const ErrorReport& err, const tc::CompilerOptions& opts = tc::CompilerOptions()) {
  if (opts.emitWarnings) std::cerr << "WARNING: " << err.what();
}

#define TC_ASSERT(ctx, cond)                                                                     \
  if (!(cond)) {                                                                                 \
    throw ::lang::ErrorReport(ctx) << __FILE__ << ":" << __LINE__ << ": assertion failed: " << #cond; \
  }

}  // namespace lang
