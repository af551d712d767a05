// Process-wide switches (the reference defines them with gflags, tc/core/flags.cc:24-130).
// Each flag reads its initial value from the environment variable TC_<NAME> (upper case) and can
// be overwritten at run time; tc::parseFlags accepts the reference's --name=value spellings.
#pragma once

#include <cstdint>
#include <string>

namespace tc {

struct Flags {
  bool debug_tc_mapper = false;     // print the matched kernel family / tile of every compile
  bool dump_cuda = false;           // print executor.compiledSource after compile
  uint32_t benchmark_warmup = 10;
  uint32_t benchmark_iterations = 100;
  uint32_t tuner_profile_iterations = 10;  // launches per candidate; the median is recorded
  std::string tuner_devices = "0";
  uint64_t random_seed = 0;
  bool tuner_print_progress = false;
};

Flags& flags();
// Consumes --name=value / --name value arguments it knows; returns the unknown ones.
int parseFlags(int argc, char** argv);
uint64_t initRandomSeed();
uint64_t randomSeed();

}  // namespace tc
