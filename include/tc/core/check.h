// Throwing check macros (the reference's tc/core/check.h:75-120): a failed check throws
// std::runtime_error carrying file:line, the failed condition and whatever was streamed in.
#pragma once

#include <sstream>
#include <stdexcept>
#include <string>

namespace tc {
namespace detail {
class Checker {
 public:
  Checker(bool ok, const char* file, int line, const std::string& what) : ok_(ok) {
    if (!ok_) msg_ << "Check failed [" << file << ":" << line << "] " << what << " ";
  }
  Checker(Checker&& o) : ok_(o.ok_) { msg_ << o.msg_.str(); o.ok_ = true; }
  ~Checker() noexcept(false) {
    if (!ok_) throw std::runtime_error(msg_.str());
  }
  template <typename T>
  Checker& operator<<(const T& t) {
    if (!ok_) msg_ << t;
    return *this;
  }

 private:
  bool ok_;
  std::stringstream msg_;
};
template <typename A, typename B>
std::string describe(const char* op, const A& a, const B& b) {
  std::stringstream ss;
  ss << a << " " << op << " " << b;
  return ss.str();
}
}  // namespace detail
}  // namespace tc

#define TC_CHECK(cond) ::tc::detail::Checker(static_cast<bool>(cond), __FILE__, __LINE__, #cond)
#define TC_CHECK_OP_(op, a, b) \
  ::tc::detail::Checker(((a)op(b)), __FILE__, __LINE__, ::tc::detail::describe(#op, (a), (b)))
#define TC_CHECK_EQ(a, b) TC_CHECK_OP_(==, a, b)
#define TC_CHECK_NE(a, b) TC_CHECK_OP_(!=, a, b)
#define TC_CHECK_LT(a, b) TC_CHECK_OP_(<, a, b)
#define TC_CHECK_LE(a, b) TC_CHECK_OP_(<=, a, b)
#define TC_CHECK_GT(a, b) TC_CHECK_OP_(>, a, b)
#define TC_CHECK_GE(a, b) TC_CHECK_OP_(>=, a, b)
