// at::Tensor <-> tensor metadata (the reference's tc/aten/aten.h:28-37, aten-inl.h:79-109).
// Descriptors are built straight from sizes()/strides()/data_ptr(): no DLPack capsule, no copy of
// the data; the at::Tensor keeps owning its storage.
#pragma once

#include <ATen/ATen.h>

#include <vector>

#include "tc/core/check.h"
#include "tc/core/tensor.h"

namespace tc {
namespace aten {

inline DLDataType toDLDataType(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return DLDataType{kDLFloat, 32, 1};
    case at::kDouble: return DLDataType{kDLFloat, 64, 1};
    case at::kHalf: return DLDataType{kDLFloat, 16, 1};
    case at::kInt: return DLDataType{kDLInt, 32, 1};
    case at::kLong: return DLDataType{kDLInt, 64, 1};
    case at::kShort: return DLDataType{kDLInt, 16, 1};
    case at::kChar: return DLDataType{kDLInt, 8, 1};
    case at::kByte: return DLDataType{kDLUInt, 8, 1};
    case at::kBool: return DLDataType{kDLUInt, 1, 1};
    default: TC_CHECK(false) << "unsupported at::ScalarType " << (int)t; return DLDataType{kDLFloat, 32, 1};
  }
}

inline at::ScalarType toScalarType(const DLDataType& t) {
  if (t.code == kDLFloat) return t.bits == 64 ? at::kDouble : t.bits == 16 ? at::kHalf : at::kFloat;
  if (t.code == kDLInt) return t.bits == 64 ? at::kLong : t.bits == 16 ? at::kShort : t.bits == 8 ? at::kChar : at::kInt;
  return t.bits == 1 ? at::kBool : at::kByte;
}

inline DLDevice toDLDevice(const at::Tensor& t) {
  return t.is_cuda() ? DLDevice{kDLCUDA, (int32_t)t.get_device()} : DLDevice{kDLCPU, 0};
}

inline TensorInfo toTensorInfo(const at::Tensor& t) {
  return TensorInfo(toDLDataType(t.scalar_type()), 0, t.sizes().vec(), t.strides().vec());
}

inline DLConstTensorUPtr makeDLConstTensor(const at::Tensor& t) {
  return tc::makeDLConstTensor(toDLDataType(t.scalar_type()), toDLDevice(t), t.sizes().vec(),
                               t.strides().vec(), t.data_ptr());
}
inline DLTensorUPtr makeDLTensor(const at::Tensor& t) {
  return tc::makeDLTensor(toDLDataType(t.scalar_type()), toDLDevice(t), t.sizes().vec(), t.strides().vec(),
                          t.data_ptr());
}
inline std::vector<DLConstTensorUPtr> makeDLConstTensors(const std::vector<at::Tensor>& ts) {
  std::vector<DLConstTensorUPtr> r;
  for (const auto& t : ts) r.push_back(makeDLConstTensor(t));
  return r;
}
inline std::vector<DLTensorUPtr> makeDLTensors(const std::vector<at::Tensor>& ts) {
  std::vector<DLTensorUPtr> r;
  for (const auto& t : ts) r.push_back(makeDLTensor(t));
  return r;
}

inline void setAtenSeed(uint64_t seed, at::Backend = at::Backend::CUDA) { at::manual_seed(seed); }

}  // namespace aten
}  // namespace tc
