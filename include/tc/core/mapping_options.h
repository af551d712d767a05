// Backend-agnostic part of the mapping options (the reference's tc/core/mapping_options.h):
// tiling, unroll factor, scheduler fusion strategies.  A plain value type with the reference's
// fluent setters; there is no protobuf underneath.
#pragma once

#include <cstdint>
#include <initializer_list>
#include <ostream>
#include <string>
#include <vector>

namespace tc {

enum class FusionStrategy { Preserve3Coincident = 0, Max = 1, Min = 2 };
std::string toString(FusionStrategy fs);
bool fromString(const std::string& s, FusionStrategy* fs);

struct SchedulerOptions {
  FusionStrategy fusionStrategy = FusionStrategy::Preserve3Coincident;
  bool allowSkewing = false;
  bool positiveOrthant = true;
  bool operator==(const SchedulerOptions& o) const {
    return fusionStrategy == o.fusionStrategy && allowSkewing == o.allowSkewing &&
           positiveOrthant == o.positiveOrthant;
  }
};

std::vector<uint64_t> parseCommaSeparatedIntegers(const std::string& s);
std::string toCommaSeparatedString(const std::vector<uint64_t>& v);

struct MappingOptions {
  std::vector<uint64_t> tiling;
  bool hasUnroll = false;
  uint64_t unrollFactor = 1;
  bool fixParametersBeforeSchedulingFlag = false;
  bool tileImperfectlyNestedFlag = false;
  bool matchLibraryCallsFlag = false;
  SchedulerOptions outerScheduleOptions, intraTileScheduleOptions;

  MappingOptions& tile(const std::vector<uint64_t>& sizes) { tiling = sizes; return *this; }
  MappingOptions& tile(std::initializer_list<uint64_t> sizes) { tiling = sizes; return *this; }
  MappingOptions& tile(const std::string& commaSeparated) { tiling = parseCommaSeparatedIntegers(commaSeparated); return *this; }
  MappingOptions& tile(const char* commaSeparated) { return tile(std::string(commaSeparated)); }
  template <typename... Args>
  MappingOptions& tile(uint64_t first, Args... rest) {
    tiling = std::vector<uint64_t>{first, static_cast<uint64_t>(rest)...};
    return *this;
  }
  MappingOptions& unroll(uint64_t size) { hasUnroll = true; unrollFactor = size; return *this; }
  MappingOptions& fixParametersBeforeScheduling(bool b) { fixParametersBeforeSchedulingFlag = b; return *this; }
  MappingOptions& tileImperfectlyNested(bool b) { tileImperfectlyNestedFlag = b; return *this; }
  MappingOptions& matchLibraryCalls(bool b) { matchLibraryCallsFlag = b; return *this; }
  MappingOptions& scheduleFusionStrategy(FusionStrategy fs) { outerScheduleOptions.fusionStrategy = fs; intraTileScheduleOptions.fusionStrategy = fs; return *this; }
  MappingOptions& scheduleFusionStrategy(const std::string& s);
  MappingOptions& outerScheduleFusionStrategy(FusionStrategy fs) { outerScheduleOptions.fusionStrategy = fs; return *this; }
  MappingOptions& outerScheduleFusionStrategy(const std::string& s);
  MappingOptions& outerScheduleAllowSkewing(bool b) { outerScheduleOptions.allowSkewing = b; return *this; }
  MappingOptions& outerSchedulePositiveOrthant(bool b) { outerScheduleOptions.positiveOrthant = b; return *this; }
  MappingOptions& intraTileScheduleFusionStrategy(FusionStrategy fs) { intraTileScheduleOptions.fusionStrategy = fs; return *this; }
  MappingOptions& intraTileScheduleFusionStrategy(const std::string& s);
  MappingOptions& intraTileScheduleAllowSkewing(bool b) { intraTileScheduleOptions.allowSkewing = b; return *this; }
  MappingOptions& intraTileSchedulePositiveOrthant(bool b) { intraTileScheduleOptions.positiveOrthant = b; return *this; }

  bool operator==(const MappingOptions& o) const;
  bool operator!=(const MappingOptions& o) const { return !(*this == o); }
  static MappingOptions makeUnmappedMappingOptions();
};

std::ostream& operator<<(std::ostream& os, const MappingOptions& o);

}  // namespace tc
