// Per-call front-end switches (the reference's tc/utils/compiler_options.h:27-37).
#pragma once

namespace tc {
struct CompilerOptions {
  bool emitWarnings = true;    // print front-end warnings to stderr
  bool throwWarnings = false;  // turn them into lang::ErrorReport exceptions
};
}  // namespace tc
