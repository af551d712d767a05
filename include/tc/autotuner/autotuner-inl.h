#pragma once

#include <algorithm>
#include <fstream>
#include <sstream>

#include "tc/core/compiler.h"
#include "tc/core/cuda/cuda_tc_executor.h"

namespace tc {
namespace autotune {

template <typename Backend>
std::string OptionsCache<Backend>::makeKey(const lang::CanonicalTcString& tc,
                                           const std::vector<TensorInfo>& inputs,
                                           const std::vector<TensorInfo>& outputs,
                                           const std::string& deviceStr) {
  std::stringstream ss;
  ss << deviceStr << "|";
  for (const auto& t : inputs) ss << t << ";";
  ss << "|";
  for (const auto& t : outputs) ss << t << ";";
  ss << "|" << tc;
  std::string k = ss.str();
  std::replace(k.begin(), k.end(), '\n', ' ');
  return k;
}

template <typename Backend>
void OptionsCache<Backend>::recordRuntime(const lang::CanonicalTcString& tc,
                                          const std::vector<TensorInfo>& inputs,
                                          const std::vector<TensorInfo>& outputs,
                                          const std::string& deviceStr, const MappingOptionsType& options,
                                          Duration runtime) {
  std::lock_guard<std::mutex> lock(mu_);
  auto& v = entries_[makeKey(tc, inputs, outputs, deviceStr)];
  const std::string ser = options.toSerializedString();
  for (auto& e : v)
    if (e.serializedOptions == ser) {
      e.runtimesUs.push_back(runtime.toMicroSeconds());
      return;
    }
  v.push_back(Entry{ser, {runtime.toMicroSeconds()}});
}

template <typename Backend>
std::vector<typename Backend::MappingOptionsType> OptionsCache<Backend>::getTopKOptions(
    const lang::CanonicalTcString& tc, const std::vector<TensorInfo>& inputs,
    const std::vector<TensorInfo>& outputs, const std::string& deviceStr, size_t k) const {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = entries_.find(makeKey(tc, inputs, outputs, deviceStr));
  if (it == entries_.end()) return {};
  std::vector<std::pair<size_t, const Entry*>> ranked;
  for (const auto& e : it->second) {
    std::vector<size_t> r = e.runtimesUs;
    std::sort(r.begin(), r.end());
    ranked.emplace_back(r[r.size() / 2], &e);
  }
  std::stable_sort(ranked.begin(), ranked.end(),
                   [](const auto& a, const auto& b) { return a.first < b.first; });
  std::vector<MappingOptionsType> out;
  for (size_t i = 0; i < ranked.size() && i < k; ++i)
    out.emplace_back(MappingOptionsType(ranked[i].second->serializedOptions));
  return out;
}

template <typename Backend>
size_t OptionsCache<Backend>::size() const {
  std::lock_guard<std::mutex> lock(mu_);
  size_t n = 0;
  for (const auto& kv : entries_) n += kv.second.size();
  return n;
}

template <typename Backend>
void OptionsCache<Backend>::clear() {
  std::lock_guard<std::mutex> lock(mu_);
  entries_.clear();
}

// File format: one line per entry, TAB separated: key, serialized options, comma separated us.
template <typename Backend>
size_t OptionsCache<Backend>::storeToFile(const std::string& filename) const {
  std::lock_guard<std::mutex> lock(mu_);
  std::ofstream out(filename, std::ios::trunc);
  size_t n = 0;
  for (const auto& kv : entries_)
    for (const auto& e : kv.second) {
      out << kv.first << "\t" << e.serializedOptions << "\t";
      for (size_t i = 0; i < e.runtimesUs.size(); ++i) out << (i ? "," : "") << e.runtimesUs[i];
      out << "\n";
      ++n;
    }
  return n;
}

template <typename Backend>
size_t OptionsCache<Backend>::loadFromFile(const std::string& filename) {
  std::lock_guard<std::mutex> lock(mu_);
  std::ifstream in(filename);
  std::string line;
  size_t n = 0;
  while (std::getline(in, line)) {
    const size_t t1 = line.find('\t'), t2 = line.rfind('\t');
    if (t1 == std::string::npos || t2 == t1) continue;
    Entry e;
    e.serializedOptions = line.substr(t1 + 1, t2 - t1 - 1);
    std::stringstream rs(line.substr(t2 + 1));
    std::string tok;
    while (std::getline(rs, tok, ',')) e.runtimesUs.push_back((size_t)strtoull(tok.c_str(), nullptr, 10));
    if (e.runtimesUs.empty()) continue;
    entries_[line.substr(0, t1)].push_back(std::move(e));
    ++n;
  }
  return n;
}

template <typename Backend, typename SearchStrategy>
std::vector<typename Backend::MappingOptionsType> Autotuner<Backend, SearchStrategy>::tune(
    const std::string& tc, const std::string& tcEntryPoint,
    const std::unordered_map<size_t, std::vector<const DLConstTensor*>>& inputs,
    std::unordered_map<size_t, std::vector<const DLTensor*>>& outputs,
    const std::vector<MappingOptionsType>& baseMappings, size_t topK,
    const TuningParameterFixer& fixedParams) {
  (void)baseMappings;  // every family default is part of the sweep already
  if (inputs.empty()) return {};
  // lowest device id first
  size_t dev = inputs.begin()->first;
  for (const auto& kv : inputs) dev = std::min(dev, kv.first);
  const auto& in = inputs.at(dev);
  const auto& out = outputs.at(dev);
  typename Backend::WithDevice guard(dev);
  std::vector<TunedCandidate> ranked = sweepTiles(tc, tcEntryPoint, in, out, fixedParams);

  auto parsed = tc::detail::parse(tc);
  const lang::CanonicalTcString canonical = lang::canonicalTc(parsed.at(tcEntryPoint));
  const std::vector<TensorInfo> inInfo = makeTensorInfoVector(in), outInfo = makeTensorInfoVector(out);
  const std::string device = Backend::backendString();
  for (const auto& c : ranked)
    optionsCache->recordRuntime(canonical, inInfo, outInfo, device, c.options,
                                Duration::fromMicroSeconds((size_t)(c.medianUs + 0.5)));
  std::vector<MappingOptionsType> result;
  for (size_t i = 0; i < ranked.size() && i < topK; ++i) result.push_back(ranked[i].options);
  return result;
}

}  // namespace autotune
}  // namespace tc
