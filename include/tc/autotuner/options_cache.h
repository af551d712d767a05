// Tuned options memoised per (canonical TC, input / output metadata, backend string), best first by
// median runtime: the reference's OptionsCache (tc/autotuner/options_cache.h:36-188,
// options_cache-inl.h) with the same file format, a serialized CudaOptionsCacheProto
// (tc/proto/compcache.proto:19-62: parallel lists of keys and values), written and parsed by
// tc/proto/wire.h instead of generated protobuf classes.  A cache file written by the reference loads
// here and the other way round; options that do not encode a tile of this backend load as "family
// default" (see cuda_mapping_options.h).
#pragma once

#include <algorithm>
#include <fstream>
#include <iterator>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "tc/core/check.h"
#include "tc/core/tensor.h"
#include "tc/core/utils/time.h"
#include "tc/lang/canonicalize.h"
#include "tc/proto/wire.h"
#include "tcb200.h"

namespace tc {
namespace autotune {

// The reference stamps every key with the git revision it was built from (tc/version/version.h) and
// only returns entries of the same revision; this backend's entries carry its ABI version instead.
inline const std::string& cacheVersionStamp() {
  static const std::string v = "tcb200-abi-" + std::to_string(TCB200_ABI_VERSION);
  return v;
}

struct OptionsCacheKey {
  lang::CanonicalTcString id;
  std::vector<TensorInfo> inputs;
  std::vector<TensorInfo> outputs;
  std::string deviceStr;
  std::string gitVersion;

  bool operator==(const OptionsCacheKey& o) const {
    return id == o.id && deviceStr == o.deviceStr && gitVersion == o.gitVersion && inputs == o.inputs &&
           outputs == o.outputs;
  }
  std::string toProtobuf() const;  // serialized OptionsCacheKeyProto
  static OptionsCacheKey fromProtobuf(proto::Reader r);
};

template <typename Backend>
struct OptionsCacheValue {
  typename Backend::MappingOptionsType mappingOptions;
  std::vector<Duration> runtimes;

  std::string toProtobuf() const;  // serialized CudaOptionsCacheValueProto
  static OptionsCacheValue fromProtobuf(proto::Reader r);
  size_t medianUs() const {
    std::vector<size_t> us;
    for (const auto& d : runtimes) us.push_back(d.toMicroSeconds());
    std::sort(us.begin(), us.end());
    return us.empty() ? ~size_t(0) : us[us.size() / 2];
  }
};

template <typename Backend>
class OptionsCache {
 public:
  using MappingOptionsType = typename Backend::MappingOptionsType;
  OptionsCache() = default;
  OptionsCache(const OptionsCache& o) {
    std::lock_guard<std::mutex> lock(o.mu_);
    store_ = o.store_;
  }

  // Adds one measured runtime for (key, options); several runtimes per options are kept.
  void recordRuntime(const lang::CanonicalTcString& tc, const std::vector<TensorInfo>& inputs,
                     const std::vector<TensorInfo>& outputs, const std::string& deviceStr,
                     const MappingOptionsType& options, Duration runtime);
  // Up to k options of the key, fastest median first (empty if the key is unknown).
  std::vector<MappingOptionsType> getTopKOptions(const lang::CanonicalTcString& tc,
                                                 const std::vector<TensorInfo>& inputs,
                                                 const std::vector<TensorInfo>& outputs,
                                                 const std::string& deviceStr, size_t k) const;
  // Drops all but the k fastest options of every key.
  void pruneKeepTopK(size_t k);
  size_t size() const;  // number of (key, options) pairs
  void clear();

  // A missing file loads as empty (options_cache-inl.h:149-157); a malformed one throws.
  void loadCacheFromFile(const std::string& filename);
  void storeCacheToFile(const std::string& filename) const;
  std::string toProtobuf() const;             // serialized CudaOptionsCacheProto
  void fromProtobuf(const std::string& bytes);  // merges into what the cache holds

 private:
  using Entry = std::pair<OptionsCacheKey, std::vector<OptionsCacheValue<Backend>>>;
  std::vector<OptionsCacheValue<Backend>>* find(const OptionsCacheKey& k);
  const std::vector<OptionsCacheValue<Backend>>* find(const OptionsCacheKey& k) const;
  void record(const OptionsCacheKey& key, const MappingOptionsType& options, Duration runtime);
  mutable std::mutex mu_;
  std::vector<Entry> store_;  // few keys per process: a linear scan keeps the key a plain struct
};

// The file-level helpers of options_cache-inl.h:336-367.
template <typename Backend>
std::vector<typename Backend::MappingOptionsType> loadTopKFromCacheFile(
    const std::string& tc, const std::string& entryPoint, const std::string& cacheFilename,
    const std::vector<const DLConstTensor*>& inputs, size_t count);
template <typename Backend>
void appendTopKToCacheFile(const OptionsCache<Backend>& cache, const std::string& cacheFilename, uint32_t count);

// ---------------------------------------------------------------------------------------------
// wire helpers: TensorInfoProto {shape 1, strides 2, alignment 3, dtype 4 {code 1, bits 2, lanes 3}}
// ---------------------------------------------------------------------------------------------
namespace detail {
inline proto::Writer tensorInfoToProto(const TensorInfo& t) {
  proto::Writer w, d;
  for (int64_t s : t.shape) w.varint(1, (uint64_t)s);
  for (int64_t s : t.strides) w.varint(2, (uint64_t)s);
  w.varint(3, t.alignment);
  d.varint(1, t.dtype.code);
  d.varint(2, t.dtype.bits);
  d.varint(3, t.dtype.lanes);
  w.message(4, d);
  return w;
}
inline TensorInfo tensorInfoFromProto(proto::Reader r) {
  DLDataType dtype{0, 0, 0};
  uint64_t alignment = 0;
  std::vector<int64_t> shape, strides;
  while (r.next()) {
    if (r.field() == 1) r.appendTo(&shape);
    else if (r.field() == 2) r.appendTo(&strides);
    else if (r.field() == 3 && r.isVarint()) alignment = r.value();
    else if (r.field() == 4 && r.isBytes()) {
      proto::Reader d = r.sub();
      while (d.next()) {
        if (!d.isVarint()) continue;
        if (d.field() == 1) dtype.code = (uint8_t)d.value();
        else if (d.field() == 2) dtype.bits = (uint8_t)d.value();
        else if (d.field() == 3) dtype.lanes = (uint16_t)d.value();
      }
      TC_CHECK(d.ok()) << "options cache: malformed dtype";
    }
  }
  TC_CHECK(r.ok()) << "options cache: malformed tensor info";
  return TensorInfo(dtype, alignment, shape, strides);
}
}  // namespace detail

// OptionsCacheKeyProto {id 1, inputs 2, outputs 3, backend_str 4, git_version 5}
inline std::string OptionsCacheKey::toProtobuf() const {
  proto::Writer w;
  w.bytes(1, id);
  for (const auto& t : inputs) w.message(2, detail::tensorInfoToProto(t));
  for (const auto& t : outputs) w.message(3, detail::tensorInfoToProto(t));
  w.bytes(4, deviceStr);
  w.bytes(5, gitVersion);
  return w.str();
}
inline OptionsCacheKey OptionsCacheKey::fromProtobuf(proto::Reader r) {
  OptionsCacheKey k;
  while (r.next()) {
    if (!r.isBytes()) continue;
    if (r.field() == 1) k.id = lang::CanonicalTcString(r.string());
    else if (r.field() == 2) k.inputs.push_back(detail::tensorInfoFromProto(r.sub()));
    else if (r.field() == 3) k.outputs.push_back(detail::tensorInfoFromProto(r.sub()));
    else if (r.field() == 4) k.deviceStr = r.string();
    else if (r.field() == 5) k.gitVersion = r.string();
  }
  TC_CHECK(r.ok()) << "options cache: malformed key";
  return k;
}

// CudaOptionsCacheValueProto {kernel_options 1, recorded_runtimes 2 (microseconds)}
template <typename Backend>
std::string OptionsCacheValue<Backend>::toProtobuf() const {
  proto::Writer w;
  w.bytes(1, mappingOptions.toProtobufSerializedString());
  for (const auto& d : runtimes) w.varint(2, d.toMicroSeconds());
  return w.str();
}
template <typename Backend>
OptionsCacheValue<Backend> OptionsCacheValue<Backend>::fromProtobuf(proto::Reader r) {
  std::string options;
  std::vector<uint64_t> us;
  bool sawOptions = false;
  while (r.next()) {
    if (r.field() == 1 && r.isBytes()) { options = r.string(); sawOptions = true; }
    else if (r.field() == 2) r.appendTo(&us);
  }
  TC_CHECK(r.ok() && sawOptions) << "options cache: malformed value";
  OptionsCacheValue v{Backend::MappingOptionsType::fromProtobufSerializedString(options), {}};
  for (uint64_t u : us) v.runtimes.push_back(Duration::fromMicroSeconds((size_t)u));
  return v;
}

template <typename Backend>
std::vector<OptionsCacheValue<Backend>>* OptionsCache<Backend>::find(const OptionsCacheKey& k) {
  for (auto& e : store_)
    if (e.first == k) return &e.second;
  return nullptr;
}
template <typename Backend>
const std::vector<OptionsCacheValue<Backend>>* OptionsCache<Backend>::find(const OptionsCacheKey& k) const {
  for (const auto& e : store_)
    if (e.first == k) return &e.second;
  return nullptr;
}

template <typename Backend>
void OptionsCache<Backend>::record(const OptionsCacheKey& key, const MappingOptionsType& options, Duration runtime) {
  auto* values = find(key);
  if (!values) {
    store_.emplace_back(key, std::vector<OptionsCacheValue<Backend>>{});
    values = &store_.back().second;
  }
  for (auto& v : *values)
    if (v.mappingOptions == options) {
      v.runtimes.push_back(runtime);
      return;
    }
  values->push_back(OptionsCacheValue<Backend>{options, {runtime}});
}

template <typename Backend>
void OptionsCache<Backend>::recordRuntime(const lang::CanonicalTcString& tc, const std::vector<TensorInfo>& inputs,
                                          const std::vector<TensorInfo>& outputs, const std::string& deviceStr,
                                          const MappingOptionsType& options, Duration runtime) {
  std::lock_guard<std::mutex> lock(mu_);
  record(OptionsCacheKey{tc, inputs, outputs, deviceStr, cacheVersionStamp()}, options, runtime);
}

template <typename Backend>
std::vector<typename Backend::MappingOptionsType> OptionsCache<Backend>::getTopKOptions(
    const lang::CanonicalTcString& tc, const std::vector<TensorInfo>& inputs, const std::vector<TensorInfo>& outputs,
    const std::string& deviceStr, size_t k) const {
  std::lock_guard<std::mutex> lock(mu_);
  const auto* values = find(OptionsCacheKey{tc, inputs, outputs, deviceStr, cacheVersionStamp()});
  if (!values) return {};
  std::vector<const OptionsCacheValue<Backend>*> ranked;
  for (const auto& v : *values) ranked.push_back(&v);
  std::stable_sort(ranked.begin(), ranked.end(), [](auto* a, auto* b) { return a->medianUs() < b->medianUs(); });
  std::vector<MappingOptionsType> out;
  for (size_t i = 0; i < ranked.size() && i < k; ++i) out.push_back(ranked[i]->mappingOptions);
  return out;
}

template <typename Backend>
void OptionsCache<Backend>::pruneKeepTopK(size_t k) {
  std::lock_guard<std::mutex> lock(mu_);
  for (auto& e : store_) {
    std::stable_sort(e.second.begin(), e.second.end(),
                     [](const auto& a, const auto& b) { return a.medianUs() < b.medianUs(); });
    if (e.second.size() > k) e.second.erase(e.second.begin() + (long)k, e.second.end());
  }
}

template <typename Backend>
size_t OptionsCache<Backend>::size() const {
  std::lock_guard<std::mutex> lock(mu_);
  size_t n = 0;
  for (const auto& e : store_) n += e.second.size();
  return n;
}

template <typename Backend>
void OptionsCache<Backend>::clear() {
  std::lock_guard<std::mutex> lock(mu_);
  store_.clear();
}

// CudaOptionsCacheProto {keys 1, values 2}: a multimap stored as parallel lists, the key repeated for
// every value (compcache.proto:47-62).
template <typename Backend>
std::string OptionsCache<Backend>::toProtobuf() const {
  std::lock_guard<std::mutex> lock(mu_);
  proto::Writer w;
  for (const auto& e : store_)
    for (size_t i = 0; i < e.second.size(); ++i) w.bytes(1, e.first.toProtobuf());
  for (const auto& e : store_)
    for (const auto& v : e.second) w.bytes(2, v.toProtobuf());
  return w.str();
}

template <typename Backend>
void OptionsCache<Backend>::fromProtobuf(const std::string& bytes) {
  std::vector<OptionsCacheKey> keys;
  std::vector<OptionsCacheValue<Backend>> values;
  proto::Reader r(bytes);
  while (r.next()) {
    if (r.field() == 1 && r.isBytes()) keys.push_back(OptionsCacheKey::fromProtobuf(r.sub()));
    else if (r.field() == 2 && r.isBytes()) values.push_back(OptionsCacheValue<Backend>::fromProtobuf(r.sub()));
  }
  TC_CHECK(r.ok()) << "options cache: malformed file";
  TC_CHECK_EQ(keys.size(), values.size()) << "options cache: keys and values do not pair up";
  std::lock_guard<std::mutex> lock(mu_);
  for (size_t i = 0; i < keys.size(); ++i)
    for (const auto& d : values[i].runtimes) record(keys[i], values[i].mappingOptions, d);
}

template <typename Backend>
void OptionsCache<Backend>::loadCacheFromFile(const std::string& filename) {
  std::ifstream in(filename, std::ios::binary);
  if (!in.is_open()) return;
  const std::string bytes((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
  fromProtobuf(bytes);
}

template <typename Backend>
void OptionsCache<Backend>::storeCacheToFile(const std::string& filename) const {
  const std::string bytes = toProtobuf();
  std::ofstream out(filename, std::ios::binary | std::ios::trunc);
  TC_CHECK(out.is_open()) << "Failed to open the output stream for dumping protobuf: " << filename;
  out.write(bytes.data(), (std::streamsize)bytes.size());
}

}  // namespace autotune
}  // namespace tc
