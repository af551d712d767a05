// tc/library/common.h of the reference: the placeholder substitution its library texts use.
#pragma once

#include <string>

namespace tc {

// Every occurrence of `search` in `str` becomes `replace` (scanning resumes after the inserted text,
// so a replacement that contains the search string is not expanded again).
inline std::string replaceString(std::string str, const std::string& search, const std::string& replace) {
  if (search.empty()) return str;
  for (size_t at = str.find(search); at != std::string::npos; at = str.find(search, at + replace.size()))
    str.replace(at, search.size(), replace);
  return str;
}

}  // namespace tc
