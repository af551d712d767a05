// Alpha-renaming of a sema-checked def: identifiers become i0, i1, ... in order of first
// appearance, so two TCs that differ only in names print identically.  The printed form is the
// key under which tuned tile configurations are memoised (the reference keys its options cache the
// same way, tc/lang/canonicalize.h:29-73).
#pragma once

#include <string>

#include "tc/lang/parser.h"
#include "tc/lang/sema.h"

namespace lang {

TreeRef canonicalize(const TreeRef& checkedDef);

struct CanonicalTcString : public std::string {
  explicit CanonicalTcString(const std::string& s = "") : std::string(s) {}
};
CanonicalTcString canonicalTc(const TreeRef& parsedDef);
CanonicalTcString canonicalTc(const std::string& tc);

}  // namespace lang
