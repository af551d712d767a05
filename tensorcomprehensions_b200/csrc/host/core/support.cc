// Tensor metadata helpers, flags, mapping options, device helpers.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <sstream>

#include "tc/core/check.h"
#include "tc/core/cuda/cuda.h"
#include "tc/core/cuda/cuda_mapping_options.h"
#include "tc/core/flags.h"
#include "tc/core/mapping_options.h"
#include "tc/core/tensor.h"
#include "tc/proto/wire.h"

namespace tc {

// ------------------------------------------------------------------------------------ tensors
TensorInfo::TensorInfo(const DLTensor* t)
    : dtype(t->dtype), alignment(0), shape(t->shape, t->shape + t->ndim) {
  strides = t->strides ? std::vector<int64_t>(t->strides, t->strides + t->ndim)
                       : makeStridesFromSizes(shape);
}
TensorInfo::TensorInfo(const DLConstTensor* t)
    : dtype(t->dtype), alignment(0), shape(t->shape, t->shape + t->ndim) {
  strides = t->strides ? std::vector<int64_t>(t->strides, t->strides + t->ndim)
                       : makeStridesFromSizes(shape);
}
bool TensorInfo::operator==(const TensorInfo& o) const {
  return dtype == o.dtype && alignment == o.alignment && shape == o.shape && strides == o.strides;
}
int64_t TensorInfo::numel() const {
  int64_t n = 1;
  for (int64_t s : shape) n *= s;
  return n;
}
bool TensorInfo::isContiguous() const {
  int64_t expect = 1;
  for (int i = (int)shape.size() - 1; i >= 0; --i) {
    if (shape[i] != 1 && strides[i] != expect) return false;
    expect *= shape[i];
  }
  return true;
}

std::vector<const DLConstTensor*> extractRawPtrs(const std::vector<DLConstTensorUPtr>& u) {
  std::vector<const DLConstTensor*> r;
  for (const auto& p : u) r.push_back(p.get());
  return r;
}
std::vector<const DLTensor*> extractRawPtrs(const std::vector<DLTensorUPtr>& u) {
  std::vector<const DLTensor*> r;
  for (const auto& p : u) r.push_back(p.get());
  return r;
}

DLDevice getCPUDLContext() { return DLDevice{kDLCPU, 0}; }
DLDevice getGPUDLContext(int id) { return DLDevice{kDLCUDA, id}; }
bool operator==(const DLDataType& a, const DLDataType& b) {
  return a.code == b.code && a.bits == b.bits && a.lanes == b.lanes;
}
std::string toString(const DLDataType& t) {
  std::stringstream ss;
  ss << (t.code == kDLFloat ? "float" : t.code == kDLInt ? "int" : t.code == kDLUInt ? "uint" : "type")
     << (int)t.bits;
  if (t.lanes > 1) ss << "x" << t.lanes;
  return ss.str();
}
std::ostream& operator<<(std::ostream& os, const DLDataType& t) { return os << toString(t); }

namespace {
template <typename T>
void printTensor(std::ostream& os, const T& t) {
  os << "DLTensor(@" << t.data << ", dim=" << t.ndim << ", type=" << t.dtype << ", sizes=[";
  for (int i = 0; i < t.ndim; ++i) os << (i ? ", " : "") << t.shape[i];
  os << "], strides=[";
  for (int i = 0; i < t.ndim; ++i) os << (i ? ", " : "") << (t.strides ? t.strides[i] : -1);
  os << "])";
}
template <typename T, typename P>
T* allocDescriptor(DLDataType dtype, DLDevice dev, const std::vector<int64_t>& sizes,
                   const std::vector<int64_t>& strides, P data) {
  T* t = new T();
  t->data = data;
  t->device = dev;
  t->ndim = (int)sizes.size();
  t->dtype = dtype;
  t->shape = new int64_t[sizes.size() ? sizes.size() : 1];
  t->strides = new int64_t[sizes.size() ? sizes.size() : 1];
  std::copy(sizes.begin(), sizes.end(), t->shape);
  std::copy(strides.begin(), strides.end(), t->strides);
  t->byte_offset = 0;
  return t;
}
}  // namespace
std::ostream& operator<<(std::ostream& os, const DLTensor& t) { printTensor(os, t); return os; }
std::ostream& operator<<(std::ostream& os, const DLConstTensor& t) { printTensor(os, t); return os; }
std::ostream& operator<<(std::ostream& os, const TensorInfo& t) {
  os << "TensorInfo(type=" << t.dtype << ", sizes=[";
  for (size_t i = 0; i < t.shape.size(); ++i) os << (i ? ", " : "") << t.shape[i];
  os << "], strides=[";
  for (size_t i = 0; i < t.strides.size(); ++i) os << (i ? ", " : "") << t.strides[i];
  return os << "])";
}

DLTensorUPtr makeDLTensor(DLDataType dtype, DLDevice dev, const std::vector<int64_t>& sizes,
                          const std::vector<int64_t>& strides, void* data) {
  return DLTensorUPtr(allocDescriptor<DLTensor>(dtype, dev, sizes, strides, data));
}
DLConstTensorUPtr makeDLConstTensor(DLDataType dtype, DLDevice dev, const std::vector<int64_t>& sizes,
                                    const std::vector<int64_t>& strides, const void* data) {
  return DLConstTensorUPtr(allocDescriptor<DLConstTensor>(dtype, dev, sizes, strides, data));
}
DLTensorUPtr makeDLTensor(const TensorInfo& i, void* data, DLDevice dev) {
  return makeDLTensor(i.dtype, dev, i.shape, i.strides, data);
}
DLConstTensorUPtr makeDLConstTensor(const TensorInfo& i, const void* data, DLDevice dev) {
  return makeDLConstTensor(i.dtype, dev, i.shape, i.strides, data);
}

// ------------------------------------------------------------------------------------ flags
namespace {
bool envBool(const char* name, bool dflt) {
  const char* v = getenv(name);
  if (!v) return dflt;
  return !(v[0] == '0' || v[0] == 'f' || v[0] == 'F' || v[0] == 'n' || v[0] == 'N' || v[0] == '\0');
}
uint64_t envU64(const char* name, uint64_t dflt) {
  const char* v = getenv(name);
  return v ? strtoull(v, nullptr, 10) : dflt;
}
uint64_t g_seed = 0;
bool g_seed_init = false;
}  // namespace

Flags& flags() {
  static Flags f = [] {
    Flags x;
    x.debug_tc_mapper = envBool("TC_DEBUG_TC_MAPPER", false);
    x.dump_cuda = envBool("TC_DUMP_CUDA", false);
    x.benchmark_warmup = (uint32_t)envU64("TC_BENCHMARK_WARMUP", 10);
    x.benchmark_iterations = (uint32_t)envU64("TC_BENCHMARK_ITERATIONS", 100);
    x.tuner_profile_iterations = (uint32_t)envU64("TC_TUNER_PROFILE_ITERATIONS", 10);
    if (const char* d = getenv("TC_TUNER_DEVICES")) x.tuner_devices = d;
    x.random_seed = envU64("TC_RANDOM_SEED", 0);
    x.tuner_print_progress = envBool("TC_TUNER_PRINT_PROGRESS", false);
    return x;
  }();
  return f;
}

int parseFlags(int argc, char** argv) {
  int kept = 1;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    bool used = false;
    if (a.rfind("--", 0) == 0) {
      std::string name = a.substr(2), value;
      const size_t eq = name.find('=');
      if (eq != std::string::npos) {
        value = name.substr(eq + 1);
        name = name.substr(0, eq);
      } else if (i + 1 < argc && argv[i + 1][0] != '-') {
        value = argv[i + 1];
      } else {
        value = "true";
      }
      const bool b = !(value == "false" || value == "0");
      Flags& f = flags();
      used = true;
      if (name == "debug_tc_mapper") f.debug_tc_mapper = b;
      else if (name == "dump_cuda") f.dump_cuda = b;
      else if (name == "benchmark_warmup") f.benchmark_warmup = (uint32_t)strtoul(value.c_str(), nullptr, 10);
      else if (name == "benchmark_iterations") f.benchmark_iterations = (uint32_t)strtoul(value.c_str(), nullptr, 10);
      else if (name == "tuner_profile_iterations") f.tuner_profile_iterations = (uint32_t)strtoul(value.c_str(), nullptr, 10);
      else if (name == "tuner_devices") f.tuner_devices = value;
      else if (name == "random_seed") f.random_seed = strtoull(value.c_str(), nullptr, 10);
      else if (name == "tuner_print_progress") f.tuner_print_progress = b;
      else used = false;
      if (used && eq == std::string::npos && value == argv[std::min(i + 1, argc - 1)] && i + 1 < argc &&
          argv[i + 1][0] != '-')
        ++i;
    }
    if (!used) argv[kept++] = argv[i];
  }
  return kept;
}

uint64_t initRandomSeed() {
  // like the reference (tc/core/flags.cc:132-144): --random_seed or wall clock, mod a prime
  if (!g_seed_init) {
    const uint64_t base = flags().random_seed ? flags().random_seed : (uint64_t)time(nullptr);
    g_seed = base % 15485863ull;
    g_seed_init = true;
  }
  return g_seed;
}
uint64_t randomSeed() { return g_seed; }

// ------------------------------------------------------------------------------------ mapping options
std::string toString(FusionStrategy fs) {
  switch (fs) {
    case FusionStrategy::Max: return "Max";
    case FusionStrategy::Min: return "Min";
    default: return "Preserve3Coincident";
  }
}
bool fromString(const std::string& s, FusionStrategy* fs) {
  if (s == "Max") *fs = FusionStrategy::Max;
  else if (s == "Min") *fs = FusionStrategy::Min;
  else if (s == "Preserve3Coincident") *fs = FusionStrategy::Preserve3Coincident;
  else return false;
  return true;
}

std::vector<uint64_t> parseCommaSeparatedIntegers(const std::string& s) {
  std::vector<uint64_t> r;
  std::stringstream ss(s);
  std::string item;
  while (std::getline(ss, item, ',')) {
    size_t b = item.find_first_not_of(" \t");
    if (b == std::string::npos) continue;
    char* end = nullptr;
    const unsigned long long v = strtoull(item.c_str() + b, &end, 10);
    TC_CHECK(end != item.c_str() + b) << "expected a comma-separated list of integers, got \"" << s << "\"";
    r.push_back(v);
  }
  return r;
}
std::string toCommaSeparatedString(const std::vector<uint64_t>& v) {
  std::stringstream ss;
  for (size_t i = 0; i < v.size(); ++i) ss << (i ? ", " : "") << v[i];
  return ss.str();
}

namespace {
FusionStrategy parseFs(const std::string& s) {
  FusionStrategy fs;
  TC_CHECK(fromString(s, &fs)) << "unknown fusion strategy " << s;
  return fs;
}
}  // namespace
MappingOptions& MappingOptions::scheduleFusionStrategy(const std::string& s) { return scheduleFusionStrategy(parseFs(s)); }
MappingOptions& MappingOptions::outerScheduleFusionStrategy(const std::string& s) { return outerScheduleFusionStrategy(parseFs(s)); }
MappingOptions& MappingOptions::intraTileScheduleFusionStrategy(const std::string& s) { return intraTileScheduleFusionStrategy(parseFs(s)); }

bool MappingOptions::operator==(const MappingOptions& o) const {
  return tiling == o.tiling && hasUnroll == o.hasUnroll && (!hasUnroll || unrollFactor == o.unrollFactor) &&
         fixParametersBeforeSchedulingFlag == o.fixParametersBeforeSchedulingFlag &&
         tileImperfectlyNestedFlag == o.tileImperfectlyNestedFlag &&
         matchLibraryCallsFlag == o.matchLibraryCallsFlag &&
         outerScheduleOptions == o.outerScheduleOptions &&
         intraTileScheduleOptions == o.intraTileScheduleOptions;
}

MappingOptions MappingOptions::makeUnmappedMappingOptions() {
  MappingOptions mo;
  mo.outerScheduleFusionStrategy(FusionStrategy::Preserve3Coincident)
      .outerScheduleAllowSkewing(false)
      .outerSchedulePositiveOrthant(true)
      .intraTileScheduleFusionStrategy(FusionStrategy::Preserve3Coincident)
      .intraTileScheduleAllowSkewing(false)
      .intraTileSchedulePositiveOrthant(true)
      .fixParametersBeforeScheduling(false)
      .tileImperfectlyNested(false)
      .matchLibraryCalls(false);
  return mo;
}

std::ostream& operator<<(std::ostream& os, const MappingOptions& o) {
  auto sched = [&](const char* name, const SchedulerOptions& s) {
    os << name << " {\n  fusion_strategy: " << toString(s.fusionStrategy)
       << "\n  allow_skewing: " << (s.allowSkewing ? "true" : "false")
       << "\n  positive_orthant: " << (s.positiveOrthant ? "true" : "false") << "\n}\n";
  };
  sched("outer_schedule_options", o.outerScheduleOptions);
  sched("intra_tile_schedule_options", o.intraTileScheduleOptions);
  os << "fix_parameters_before_scheduling: " << (o.fixParametersBeforeSchedulingFlag ? "true" : "false") << "\n";
  if (!o.tiling.empty()) {
    os << "tiling {\n";
    for (auto t : o.tiling) os << "  sizes: " << t << "\n";
    os << "}\n";
  }
  if (o.hasUnroll) os << "unroll: " << o.unrollFactor << "\n";
  os << "tile_imperfectly_nested: " << (o.tileImperfectlyNestedFlag ? "true" : "false") << "\n";
  os << "match_library_calls: " << (o.matchLibraryCallsFlag ? "true" : "false") << "\n";
  return os;
}

CudaDim::CudaDim(std::initializer_list<uint64_t> il) : CudaDim(std::vector<uint64_t>(il)) {}
CudaDim::CudaDim(const std::vector<uint64_t>& v) {
  TC_CHECK_GT(v.size(), 0u) << "list of values in CudaDim must be non-empty";
  TC_CHECK_LE(v.size(), 3u) << "at most 3 values allowed in CudaDim";
  x = v[0];
  y = v.size() > 1 ? v[1] : defaultDim;
  z = v.size() > 2 ? v[2] : defaultDim;
}
std::string CudaDim::toCommaSeparatedString() const {
  std::stringstream ss;
  ss << x;
  if (y != defaultDim || z != defaultDim) ss << ", " << y;
  if (z != defaultDim) ss << ", " << z;
  return ss.str();
}
std::ostream& operator<<(std::ostream& os, const CudaDim& d) {
  return os << "CudaDim(" << d.toCommaSeparatedString() << ")";
}

CudaMappingOptions& CudaMappingOptions::mapToThreads(const std::string& s) {
  auto v = parseCommaSeparatedIntegers(s);
  TC_CHECK_GT(v.size(), 0u) << "expected at least one block size in " << s;
  TC_CHECK_LE(v.size(), 3u) << "expected at most three block sizes in " << s;
  return mapToThreads(v);
}
CudaMappingOptions& CudaMappingOptions::mapToBlocks(const std::string& s) {
  auto v = parseCommaSeparatedIntegers(s);
  TC_CHECK_GT(v.size(), 0u) << "expected at least one grid size in " << s;
  TC_CHECK_LE(v.size(), 3u) << "expected at most three grid sizes in " << s;
  return mapToBlocks(v);
}

bool CudaMappingOptions::operator==(const CudaMappingOptions& o) const {
  return generic == o.generic && block == o.block && grid == o.grid &&
         useSharedMemoryFlag == o.useSharedMemoryFlag && usePrivateMemoryFlag == o.usePrivateMemoryFlag &&
         unrollCopySharedFlag == o.unrollCopySharedFlag && useReadOnlyCacheFlag == o.useReadOnlyCacheFlag &&
         hasMaxSharedMemory == o.hasMaxSharedMemory &&
         (!hasMaxSharedMemory || maxSharedMemoryBytes == o.maxSharedMemoryBytes) &&
         privateDepthValue == o.privateDepthValue && sharedDepthValue == o.sharedDepthValue;
}

CudaMappingOptions CudaMappingOptions::makeUnmappedMappingOptions() {
  CudaMappingOptions mo;
  mo.genericMappingOptions(MappingOptions::makeUnmappedMappingOptions())
      .useSharedMemory(false).usePrivateMemory(false).unrollCopyShared(false).useReadOnlyCache(false);
  return mo;
}
// Preset values as in the reference (tc/core/cuda/cuda_mapping_options.cc:337-384); to this
// backend every preset means "family default tile".
CudaMappingOptions CudaMappingOptions::makeNaiveMappingOptions() {
  return makeUnmappedMappingOptions().tile(32, 32, 32).mapToThreads(32, 8).mapToBlocks(256, 256).unroll(1);
}
CudaMappingOptions CudaMappingOptions::makeSingleThreadMappingOptions() {
  return makeUnmappedMappingOptions().tile(1).mapToThreads(1).mapToBlocks(1).unroll(1);
}
CudaMappingOptions CudaMappingOptions::makePointwiseMappingOptions() {
  return makeUnmappedMappingOptions().tile(32, 32, 32).mapToThreads(32, 4, 4).mapToBlocks(100, 100, 100).unroll(128);
}
CudaMappingOptions CudaMappingOptions::makeMlpMappingOptions() {
  return makeUnmappedMappingOptions().outerScheduleFusionStrategy(FusionStrategy::Max).tile(1).mapToThreads(128).mapToBlocks(128).unroll(1);
}
CudaMappingOptions CudaMappingOptions::makeConvolutionMappingOptions() {
  return makeUnmappedMappingOptions().tile(4, 8, 8, 8).mapToThreads(4, 16, 4).mapToBlocks(256, 256, 256).unroll(1);
}
CudaMappingOptions CudaMappingOptions::makeGroupConvolutionMappingOptions() {
  return makeUnmappedMappingOptions().tile(1, 1).mapToThreads(4, 16, 4).mapToBlocks(256, 256).unroll(1);
}

CudaMappingOptions CudaMappingOptions::fromTile(const tcb200_tile_t& t) {
  CudaMappingOptions mo = makeUnmappedMappingOptions();
  // a fourth tile size carries the split of the reduction (split-K) when there is one
  if (t.split_k > 1) mo.tile((uint64_t)t.bm, (uint64_t)t.bn, (uint64_t)t.bk, (uint64_t)t.split_k);
  else mo.tile((uint64_t)t.bm, (uint64_t)t.bn, (uint64_t)t.bk);
  mo.mapToThreads((uint64_t)std::max(t.threads, 1))
      .mapToBlocks(1)
      .unroll((uint64_t)t.stages)
      .useSharedMemory(true)
      .usePrivateMemory(t.split_tf32 == 3)
      .matchLibraryCalls(true)
      .privateDepth((uint32_t)t.variant)
      .sharedDepth((uint32_t)t.split_tf32);
  return mo;
}
bool CudaMappingOptions::toTile(tcb200_tile_t* t) const {
  if (!generic.matchLibraryCallsFlag || (generic.tiling.size() != 3 && generic.tiling.size() != 4) ||
      privateDepthValue == 0)
    return false;
  memset(t, 0, sizeof(*t));
  t->variant = (int)privateDepthValue;
  t->bm = (int)generic.tiling[0];
  t->bn = (int)generic.tiling[1];
  t->bk = (int)generic.tiling[2];
  t->stages = generic.hasUnroll ? (int)generic.unrollFactor : 0;
  t->threads = (int)block.x;
  t->split_tf32 = (int)sharedDepthValue;
  t->split_k = generic.tiling.size() == 4 ? (int)generic.tiling[3] : 0;
  return true;
}

// text form: key=value;... (own format; enough to round-trip through a cache file)
std::string CudaMappingOptions::toSerializedString() const {
  std::stringstream ss;
  ss << "tile=" << toCommaSeparatedString(generic.tiling) << ";unroll=" << (generic.hasUnroll ? (long long)generic.unrollFactor : -1)
     << ";fix=" << generic.fixParametersBeforeSchedulingFlag << ";tin=" << generic.tileImperfectlyNestedFlag
     << ";mlc=" << generic.matchLibraryCallsFlag
     << ";ofs=" << toString(generic.outerScheduleOptions.fusionStrategy) << ";oas=" << generic.outerScheduleOptions.allowSkewing
     << ";opo=" << generic.outerScheduleOptions.positiveOrthant
     << ";ifs=" << toString(generic.intraTileScheduleOptions.fusionStrategy) << ";ias=" << generic.intraTileScheduleOptions.allowSkewing
     << ";ipo=" << generic.intraTileScheduleOptions.positiveOrthant
     << ";block=" << block.x << "," << block.y << "," << block.z << ";grid=" << grid.x << "," << grid.y << "," << grid.z
     << ";shared=" << useSharedMemoryFlag << ";private=" << usePrivateMemoryFlag << ";ucs=" << unrollCopySharedFlag
     << ";roc=" << useReadOnlyCacheFlag << ";maxshared=" << (hasMaxSharedMemory ? (long long)maxSharedMemoryBytes : -1)
     << ";pdepth=" << privateDepthValue << ";sdepth=" << sharedDepthValue;
  return ss.str();
}
// ---- CudaMappingOptionsProto on the wire (field numbers: tc/proto/mapping_options.proto:19-91) ----
namespace {
// FusionStrategy in the proto: Max = 1, Preserve3Coincident = 2, Min = 3
uint64_t fusionToProto(FusionStrategy f) {
  return f == FusionStrategy::Max ? 1 : f == FusionStrategy::Preserve3Coincident ? 2 : 3;
}
FusionStrategy fusionFromProto(uint64_t v) {
  TC_CHECK(v >= 1 && v <= 3) << "mapping options: unknown fusion strategy " << v;
  return v == 1 ? FusionStrategy::Max : v == 2 ? FusionStrategy::Preserve3Coincident : FusionStrategy::Min;
}
proto::Writer schedulerToProto(const SchedulerOptions& o) {
  proto::Writer w;
  w.varint(1, fusionToProto(o.fusionStrategy));
  w.boolean(2, o.allowSkewing);
  w.boolean(3, o.positiveOrthant);
  return w;
}
void schedulerFromProto(proto::Reader r, SchedulerOptions* o) {
  while (r.next()) {
    if (r.field() == 1 && r.isVarint()) o->fusionStrategy = fusionFromProto(r.value());
    else if (r.field() == 2 && r.isVarint()) o->allowSkewing = r.value() != 0;
    else if (r.field() == 3 && r.isVarint()) o->positiveOrthant = r.value() != 0;
  }
  TC_CHECK(r.ok()) << "mapping options: malformed scheduler options";
}
// y and z are optional in the proto (absent = not mapped); here an unmapped dimension has extent 1
proto::Writer dimToProto(const CudaDim& d) {
  proto::Writer w;
  w.varint(1, d.x);
  if (d.y != CudaDim::defaultDim || d.z != CudaDim::defaultDim) w.varint(2, d.y);
  if (d.z != CudaDim::defaultDim) w.varint(3, d.z);
  return w;
}
void dimFromProto(proto::Reader r, CudaDim* d) {
  *d = CudaDim(CudaDim::defaultDim);
  while (r.next()) {
    if (!r.isVarint()) continue;
    if (r.field() == 1) d->x = r.value();
    else if (r.field() == 2) d->y = r.value();
    else if (r.field() == 3) d->z = r.value();
  }
  TC_CHECK(r.ok()) << "mapping options: malformed block / grid";
}
}  // namespace

std::string CudaMappingOptions::toProtobufSerializedString() const {
  proto::Writer g;  // MappingOptionsProto
  g.message(1, schedulerToProto(generic.outerScheduleOptions));
  g.message(2, schedulerToProto(generic.intraTileScheduleOptions));
  g.boolean(3, generic.fixParametersBeforeSchedulingFlag);
  if (!generic.tiling.empty()) {
    proto::Writer t;
    for (uint64_t s : generic.tiling) t.varint(1, s);
    g.message(4, t);
  }
  if (generic.hasUnroll) g.varint(5, generic.unrollFactor);
  g.boolean(6, generic.tileImperfectlyNestedFlag);
  g.boolean(7, generic.matchLibraryCallsFlag);
  proto::Writer w;  // CudaMappingOptionsProto
  w.message(1, g);
  w.message(2, dimToProto(block));
  w.message(3, dimToProto(grid));
  w.boolean(4, useSharedMemoryFlag);
  w.boolean(5, usePrivateMemoryFlag);
  w.boolean(6, unrollCopySharedFlag);
  if (hasMaxSharedMemory) w.varint(7, maxSharedMemoryBytes);
  w.boolean(8, useReadOnlyCacheFlag);
  w.varint(9, privateDepthValue);
  w.varint(10, sharedDepthValue);
  return w.str();
}

CudaMappingOptions CudaMappingOptions::fromProtobufSerializedString(const std::string& bytes) {
  CudaMappingOptions o = makeUnmappedMappingOptions();
  o.generic.tiling.clear();
  o.generic.hasUnroll = false;
  o.hasMaxSharedMemory = false;
  bool sawGeneric = false, sawBlock = false, sawGrid = false;
  proto::Reader r(bytes);
  while (r.next()) {
    const uint32_t f = r.field();
    if (f == 1 && r.isBytes()) {
      sawGeneric = true;
      proto::Reader g = r.sub();
      while (g.next()) {
        const uint32_t gf = g.field();
        if (gf == 1 && g.isBytes()) schedulerFromProto(g.sub(), &o.generic.outerScheduleOptions);
        else if (gf == 2 && g.isBytes()) schedulerFromProto(g.sub(), &o.generic.intraTileScheduleOptions);
        else if (gf == 3 && g.isVarint()) o.generic.fixParametersBeforeSchedulingFlag = g.value() != 0;
        else if (gf == 4 && g.isBytes()) {
          proto::Reader t = g.sub();
          while (t.next())
            if (t.field() == 1) t.appendTo(&o.generic.tiling);
          TC_CHECK(t.ok()) << "mapping options: malformed tiling";
        } else if (gf == 5 && g.isVarint()) { o.generic.hasUnroll = true; o.generic.unrollFactor = g.value(); }
        else if (gf == 6 && g.isVarint()) o.generic.tileImperfectlyNestedFlag = g.value() != 0;
        else if (gf == 7 && g.isVarint()) o.generic.matchLibraryCallsFlag = g.value() != 0;
      }
      TC_CHECK(g.ok()) << "mapping options: malformed generic options";
    } else if (f == 2 && r.isBytes()) { sawBlock = true; dimFromProto(r.sub(), &o.block); }
    else if (f == 3 && r.isBytes()) { sawGrid = true; dimFromProto(r.sub(), &o.grid); }
    else if (f == 4 && r.isVarint()) o.useSharedMemoryFlag = r.value() != 0;
    else if (f == 5 && r.isVarint()) o.usePrivateMemoryFlag = r.value() != 0;
    else if (f == 6 && r.isVarint()) o.unrollCopySharedFlag = r.value() != 0;
    else if (f == 7 && r.isVarint()) { o.hasMaxSharedMemory = true; o.maxSharedMemoryBytes = r.value(); }
    else if (f == 8 && r.isVarint()) o.useReadOnlyCacheFlag = r.value() != 0;
    else if (f == 9 && r.isVarint()) o.privateDepthValue = (uint32_t)r.value();
    else if (f == 10 && r.isVarint()) o.sharedDepthValue = (uint32_t)r.value();
  }
  TC_CHECK(r.ok() && sawGeneric && sawBlock && sawGrid)
      << "not a serialized CudaMappingOptionsProto (required fields missing or bytes malformed)";
  return o;
}

CudaMappingOptions::CudaMappingOptions(const std::string& serialized) {
  if (serialized.compare(0, 5, "tile=") != 0) {  // not the text form: protobuf bytes
    *this = fromProtobufSerializedString(serialized);
    return;
  }
  *this = makeUnmappedMappingOptions();
  std::stringstream ss(serialized);
  std::string kv;
  while (std::getline(ss, kv, ';')) {
    const size_t eq = kv.find('=');
    TC_CHECK(eq != std::string::npos) << "malformed mapping options string: " << serialized;
    const std::string k = kv.substr(0, eq), v = kv.substr(eq + 1);
    auto b = [&] { return v == "1"; };
    if (k == "tile") generic.tiling = parseCommaSeparatedIntegers(v);
    else if (k == "unroll") { long long u = atoll(v.c_str()); generic.hasUnroll = u >= 0; generic.unrollFactor = u >= 0 ? u : 1; }
    else if (k == "fix") generic.fixParametersBeforeSchedulingFlag = b();
    else if (k == "tin") generic.tileImperfectlyNestedFlag = b();
    else if (k == "mlc") generic.matchLibraryCallsFlag = b();
    else if (k == "ofs") generic.outerScheduleOptions.fusionStrategy = parseFs(v);
    else if (k == "oas") generic.outerScheduleOptions.allowSkewing = b();
    else if (k == "opo") generic.outerScheduleOptions.positiveOrthant = b();
    else if (k == "ifs") generic.intraTileScheduleOptions.fusionStrategy = parseFs(v);
    else if (k == "ias") generic.intraTileScheduleOptions.allowSkewing = b();
    else if (k == "ipo") generic.intraTileScheduleOptions.positiveOrthant = b();
    else if (k == "block") block = CudaDim(parseCommaSeparatedIntegers(v));
    else if (k == "grid") grid = CudaDim(parseCommaSeparatedIntegers(v));
    else if (k == "shared") useSharedMemoryFlag = b();
    else if (k == "private") usePrivateMemoryFlag = b();
    else if (k == "ucs") unrollCopySharedFlag = b();
    else if (k == "roc") useReadOnlyCacheFlag = b();
    else if (k == "maxshared") { long long m = atoll(v.c_str()); hasMaxSharedMemory = m >= 0; maxSharedMemoryBytes = m >= 0 ? m : 0; }
    else if (k == "pdepth") privateDepthValue = (uint32_t)atoll(v.c_str());
    else if (k == "sdepth") sharedDepthValue = (uint32_t)atoll(v.c_str());
    else TC_CHECK(false) << "unknown key " << k << " in mapping options string";
  }
}

std::ostream& operator<<(std::ostream& os, const CudaMappingOptions& o) {
  os << "generic_mapping_options {\n" << o.generic << "}\n";
  os << "block {\n  x: " << o.block.x << "\n  y: " << o.block.y << "\n  z: " << o.block.z << "\n}\n";
  os << "grid {\n  x: " << o.grid.x << "\n  y: " << o.grid.y << "\n  z: " << o.grid.z << "\n}\n";
  os << "use_shared_memory: " << (o.useSharedMemoryFlag ? "true" : "false") << "\n";
  os << "use_private_memory: " << (o.usePrivateMemoryFlag ? "true" : "false") << "\n";
  os << "unroll_copy_shared: " << (o.unrollCopySharedFlag ? "true" : "false") << "\n";
  os << "use_readonly_cache: " << (o.useReadOnlyCacheFlag ? "true" : "false") << "\n";
  if (o.hasMaxSharedMemory) os << "max_shared_memory: " << o.maxSharedMemoryBytes << "\n";
  os << "private_depth: " << o.privateDepthValue << "\nshared_depth: " << o.sharedDepthValue << "\n";
  tcb200_tile_t t;
  if (o.toTile(&t))
    os << "# tile sweep point: variant=" << t.variant << " tile=" << t.bm << "x" << t.bn << "x" << t.bk
       << " stages=" << t.stages << " threads=" << t.threads << " split_tf32=" << t.split_tf32 << " split_k=" << t.split_k << "\n";
  return os;
}

// ------------------------------------------------------------------------------------ device helpers
void tcb200Enforce(int status, const char* what) {
  if (status == TCB200_OK) return;
  std::stringstream ss;
  ss << "tcb200 error " << status << " (" << tcb200_strerror(status) << ") in " << what;
  if (status == TCB200_ERR_CUDA) ss << " [cudaError " << tcb200_last_cuda_error() << "]";
  throw std::runtime_error(ss.str());
}

WithCudaDevice::WithCudaDevice(size_t newDevice) {
  TC_TCB200_ENFORCE(tcb200_get_device(&oldDevice_));
  TC_TCB200_ENFORCE(tcb200_set_device((int)newDevice));
}
WithCudaDevice::~WithCudaDevice() { tcb200_set_device(oldDevice_); }

CudaGPUInfo& CudaGPUInfo::GPUInfo() {
  static thread_local CudaGPUInfo info;
  return info;
}
int CudaGPUInfo::NumberGPUs() const {
  int n = 0;
  tcb200_device_count(&n);
  return n;
}
int CudaGPUInfo::CurrentGPUId() const {
  int d = 0;
  TC_TCB200_ENFORCE(tcb200_get_device(&d));
  return d;
}
std::string CudaGPUInfo::GetGPUName(int id) const {
  if (NumberGPUs() == 0) return "no-gpu";
  if (id < 0) id = CurrentGPUId();
  char buf[256];
  TC_TCB200_ENFORCE(tcb200_device_name(id, buf, sizeof(buf)));
  return buf;
}

}  // namespace tc
