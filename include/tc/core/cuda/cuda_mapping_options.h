// CudaMappingOptions — the options type of tc::aten::compile<CudaBackend> and the element type
// ATenAutotuner::tune returns (the reference's tc/core/cuda/cuda_mapping_options.h:145-245).
//
// The type, its fluent setters and its presets are kept; what the fields MEAN to this backend is
// different, because there is no polyhedral mapper to steer.  A tuned options object encodes one
// point of a kernel family's tile sweep:
//     tile(bm, bn, bk)             CTA tile (rows of c1 per stage for tensordot)
//     mapToThreads(threads)        CTA size
//     unroll(stages)               TMA / bulk-copy pipeline depth
//     usePrivateMemory(b)          true: 3xTF32 split (fp32 accuracy); false: one TF32 pass
//     matchLibraryCalls(true)      marks the object as "tile encoded" ...
//     privateDepth(variant)        ... for this kernel variant (TCB200_VARIANT_*)
// Anything else — makeNaiveMappingOptions() and the other presets, or hand-written options from
// reference code — means "no preference": the family default tile is used.
#pragma once

#include <array>
#include <cstdint>
#include <initializer_list>
#include <ostream>
#include <string>
#include <vector>

#include "tc/core/mapping_options.h"
#include "tcb200.h"

namespace tc {

struct CudaDim {
  static constexpr uint64_t defaultDim = 1;
  uint64_t x = defaultDim, y = defaultDim, z = defaultDim;
  CudaDim() = default;
  CudaDim(uint64_t x_, uint64_t y_ = defaultDim, uint64_t z_ = defaultDim) : x(x_), y(y_), z(z_) {}
  CudaDim(std::initializer_list<uint64_t> il);
  CudaDim(const std::vector<uint64_t>& v);
  std::vector<uint64_t> extractVector() const { return {x, y, z}; }
  std::array<uint64_t, 3> extractDefaultedArray() const { return {{x, y, z}}; }
  std::string toCommaSeparatedString() const;
  bool operator==(const CudaDim& o) const { return x == o.x && y == o.y && z == o.z; }
  bool operator!=(const CudaDim& o) const { return !(*this == o); }
};
struct Block : CudaDim { using CudaDim::CudaDim; Block() = default; Block(const CudaDim& d) : CudaDim(d) {} };
struct Grid : CudaDim { using CudaDim::CudaDim; Grid() = default; Grid(const CudaDim& d) : CudaDim(d) {} };

class CudaMappingOptions {
 private:
  CudaMappingOptions() = default;
  static CudaMappingOptions makeUnmappedMappingOptions();

 public:
  CudaMappingOptions(const CudaMappingOptions&) = default;
  CudaMappingOptions& operator=(const CudaMappingOptions&) = default;
  // From toProtobufSerializedString() (a serialized CudaMappingOptionsProto, as in the reference:
  // tc/core/cuda/cuda_mapping_options.cc) or from this library's text form toSerializedString().
  explicit CudaMappingOptions(const std::string& serialized);
  bool operator==(const CudaMappingOptions& o) const;
  bool operator!=(const CudaMappingOptions& o) const { return !(*this == o); }
  std::string toSerializedString() const;
  // The wire bytes of CudaMappingOptionsProto (tc/proto/mapping_options.proto:71-91): readable by the
  // reference's generated classes and the other way round.
  std::string toProtobufSerializedString() const;
  static CudaMappingOptions fromProtobufSerializedString(const std::string& bytes);

  CudaMappingOptions& mapToThreads(std::initializer_list<uint64_t> t) { block = CudaDim(t); return *this; }
  CudaMappingOptions& mapToThreads(uint64_t x, uint64_t y = CudaDim::defaultDim, uint64_t z = CudaDim::defaultDim) { block = CudaDim(x, y, z); return *this; }
  CudaMappingOptions& mapToThreads(const std::vector<uint64_t>& t) { block = CudaDim(t); return *this; }
  CudaMappingOptions& mapToThreads(const std::string& commaSeparatedSizes);
  CudaMappingOptions& mapToBlocks(std::initializer_list<uint64_t> b) { grid = CudaDim(b); return *this; }
  CudaMappingOptions& mapToBlocks(uint64_t x, uint64_t y = CudaDim::defaultDim, uint64_t z = CudaDim::defaultDim) { grid = CudaDim(x, y, z); return *this; }
  CudaMappingOptions& mapToBlocks(const std::vector<uint64_t>& b) { grid = CudaDim(b); return *this; }
  CudaMappingOptions& mapToBlocks(const std::string& commaSeparatedSizes);
  CudaMappingOptions& genericMappingOptions(const MappingOptions& o) { generic = o; return *this; }
  CudaMappingOptions& useSharedMemory(bool b) { useSharedMemoryFlag = b; return *this; }
  CudaMappingOptions& usePrivateMemory(bool b) { usePrivateMemoryFlag = b; return *this; }
  CudaMappingOptions& maxSharedMemory(uint64_t size) { hasMaxSharedMemory = true; maxSharedMemoryBytes = size; return *this; }
  CudaMappingOptions& unrollCopyShared(bool b) { unrollCopySharedFlag = b; return *this; }
  CudaMappingOptions& useReadOnlyCache(bool b) { useReadOnlyCacheFlag = b; return *this; }
  CudaMappingOptions& privateDepth(uint32_t depth) { privateDepthValue = depth; return *this; }
  CudaMappingOptions& sharedDepth(uint32_t depth) { sharedDepthValue = depth; return *this; }

  static CudaMappingOptions makeNaiveMappingOptions();
  static CudaMappingOptions makeSingleThreadMappingOptions();
  static CudaMappingOptions makePointwiseMappingOptions();
  static CudaMappingOptions makeMlpMappingOptions();
  static CudaMappingOptions makeConvolutionMappingOptions();
  static CudaMappingOptions makeGroupConvolutionMappingOptions();

#define TC_FORWARD_GENERIC(FUN)                    \
  template <typename... Args>                      \
  CudaMappingOptions& FUN(Args... args) {          \
    generic.FUN(args...);                          \
    return *this;                                  \
  }
  TC_FORWARD_GENERIC(tile)
  TC_FORWARD_GENERIC(unroll)
  TC_FORWARD_GENERIC(fixParametersBeforeScheduling)
  TC_FORWARD_GENERIC(tileImperfectlyNested)
  TC_FORWARD_GENERIC(matchLibraryCalls)
  TC_FORWARD_GENERIC(scheduleFusionStrategy)
  TC_FORWARD_GENERIC(outerScheduleFusionStrategy)
  TC_FORWARD_GENERIC(outerScheduleAllowSkewing)
  TC_FORWARD_GENERIC(outerSchedulePositiveOrthant)
  TC_FORWARD_GENERIC(intraTileScheduleFusionStrategy)
  TC_FORWARD_GENERIC(intraTileScheduleAllowSkewing)
  TC_FORWARD_GENERIC(intraTileSchedulePositiveOrthant)
#undef TC_FORWARD_GENERIC

  // ---- the tile-sweep encoding described at the top of this file --------------------------
  static CudaMappingOptions fromTile(const tcb200_tile_t& tile);
  // True (and *tile filled) iff the object was produced by fromTile.
  bool toTile(tcb200_tile_t* tile) const;

  MappingOptions generic;
  CudaDim block, grid;
  bool useSharedMemoryFlag = false, usePrivateMemoryFlag = false, unrollCopySharedFlag = false,
       useReadOnlyCacheFlag = false, hasMaxSharedMemory = false;
  uint64_t maxSharedMemoryBytes = 0;
  uint32_t privateDepthValue = 0, sharedDepthValue = 0;
};

std::ostream& operator<<(std::ostream& os, const CudaDim& dim);
std::ostream& operator<<(std::ostream& os, const CudaMappingOptions& o);

}  // namespace tc
