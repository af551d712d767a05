// Driver around the reference's own tc/lang front-end (compiled from the
// reference's sources by `make ref`; nothing of the reference is copied here).
// TEST INFRASTRUCTURE ONLY: used to generate tests/golden/lang/* and to
// differential-test the re-written front-end in this container.
//
//   tc_lang_ref parse  file.tc   -> s-expression of every def after parsing
//   tc_lang_ref sema   file.tc   -> s-expression after Sema::checkFunction + environment dump
//   tc_lang_ref canon  file.tc   -> canonicalised (alpha-renamed) sema-checked tree of every def
// A lang::ErrorReport is printed as "ERROR: <what()>" and the exit code is 3.
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>

#include "tc/lang/canonicalize.h"
#include "tc/lang/parser.h"
#include "tc/lang/sema.h"

int main(int argc, char** argv) {
  if (argc != 3) {
    std::cerr << "usage: tc_lang_ref parse|sema|canon file.tc\n";
    return 2;
  }
  std::string mode = argv[1];
  std::ifstream in(argv[2]);
  if (!in.good()) {
    std::cerr << "cannot read " << argv[2] << "\n";
    return 2;
  }
  std::stringstream buf;
  buf << in.rdbuf();
  try {
    lang::Parser parser(buf.str());
    while (parser.L.cur().kind != lang::TK_EOF) {
      auto def = parser.parseFunction();
      if (mode == "parse") {
        std::cout << def;
      } else if (mode == "sema") {
        lang::Sema sema;
        auto checked = sema.checkFunction(def);
        std::cout << checked << sema.dumpEnv();
      } else if (mode == "canon") {
        std::cout << lang::canonicalize(lang::Sema().checkFunction(def));
      } else {
        std::cerr << "unknown mode " << mode << "\n";
        return 2;
      }
    }
  } catch (const lang::ErrorReport& e) {
    std::cout << "ERROR: " << e.what() << "\n";
    return 3;
  }
  return 0;
}
