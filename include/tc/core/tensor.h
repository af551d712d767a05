// Tensor metadata types at the API boundary (the reference's tc/core/tensor.h:46-101).
//
// Tensors cross the boundary as DLPack-style descriptors whose data pointer is BORROWED; the
// executor keeps only TensorInfo (dtype, shape, strides).  DLConstTensor mirrors DLTensor with a
// const data pointer.  The DLPack structs are declared here (layout of DLPack 1.x) unless a DLPack
// header was already included.
#pragma once

#include <cstdint>
#include <memory>
#include <ostream>
#include <string>
#include <vector>

#ifndef DLPACK_DLPACK_H_
#define DLPACK_DLPACK_H_
extern "C" {
typedef enum { kDLCPU = 1, kDLCUDA = 2, kDLCUDAHost = 3 } DLDeviceType;
typedef struct {
  DLDeviceType device_type;
  int32_t device_id;
} DLDevice;
typedef enum { kDLInt = 0U, kDLUInt = 1U, kDLFloat = 2U, kDLBfloat = 4U, kDLBool = 6U } DLDataTypeCode;
typedef struct {
  uint8_t code;
  uint8_t bits;
  uint16_t lanes;
} DLDataType;
typedef struct {
  void* data;
  DLDevice device;
  int32_t ndim;
  DLDataType dtype;
  int64_t* shape;
  int64_t* strides;
  uint64_t byte_offset;
} DLTensor;
}
#endif

typedef struct {
  const void* data;
  DLDevice device;
  int32_t ndim;
  DLDataType dtype;
  int64_t* shape;
  int64_t* strides;
  uint64_t byte_offset;
} DLConstTensor;

namespace tc {

// Owns the descriptor and its shape/stride arrays, never the data.
struct DLTensorDeleter {
  template <typename T>
  void operator()(const T* t) const {
    if (!t) return;
    delete[] t->shape;
    delete[] t->strides;
    delete t;
  }
};
using DLTensorUPtr = std::unique_ptr<DLTensor, DLTensorDeleter>;
using DLConstTensorUPtr = std::unique_ptr<DLConstTensor, DLTensorDeleter>;

std::vector<const DLConstTensor*> extractRawPtrs(const std::vector<DLConstTensorUPtr>& uptrs);
std::vector<const DLTensor*> extractRawPtrs(const std::vector<DLTensorUPtr>& uptrs);

template <typename T>
std::vector<T> makeStridesFromSizes(const std::vector<T>& sizes) {
  std::vector<T> strides(sizes.size(), 1);
  for (int i = (int)sizes.size() - 2; i >= 0; --i) strides[i] = strides[i + 1] * sizes[i + 1];
  return strides;
}

struct TensorInfo {
  static constexpr int kAlignment = 256;
  DLDataType dtype;
  uint64_t alignment;
  std::vector<int64_t> shape;
  std::vector<int64_t> strides;

  TensorInfo(DLDataType dtype, uint64_t alignment, const std::vector<int64_t>& shape,
             const std::vector<int64_t>& strides)
      : dtype(dtype), alignment(alignment), shape(shape), strides(strides) {}
  explicit TensorInfo(const DLTensor* t);
  explicit TensorInfo(const DLConstTensor* t);
  explicit TensorInfo(const DLTensorUPtr& t) : TensorInfo(t.get()) {}
  explicit TensorInfo(const DLConstTensorUPtr& t) : TensorInfo(t.get()) {}
  bool operator==(const TensorInfo& o) const;
  bool operator!=(const TensorInfo& o) const { return !(*this == o); }
  int64_t numel() const;
  bool isContiguous() const;
};

template <typename P>
std::vector<TensorInfo> makeTensorInfoVector(const std::vector<P>& ts) {
  std::vector<TensorInfo> r;
  r.reserve(ts.size());
  for (const auto& t : ts) r.emplace_back(TensorInfo(t));
  return r;
}

DLDevice getCPUDLContext();
DLDevice getGPUDLContext(int device_id = 0);
bool operator==(const DLDataType& a, const DLDataType& b);
std::string toString(const DLDataType& t);
std::ostream& operator<<(std::ostream& os, const DLDataType& t);
std::ostream& operator<<(std::ostream& os, const DLTensor& t);
std::ostream& operator<<(std::ostream& os, const DLConstTensor& t);
std::ostream& operator<<(std::ostream& os, const TensorInfo& t);

// Metadata-owning descriptors.
DLTensorUPtr makeDLTensor(const TensorInfo& info, void* data = nullptr, DLDevice dev = DLDevice{kDLCUDA, 0});
DLConstTensorUPtr makeDLConstTensor(const TensorInfo& info, const void* data = nullptr,
                                    DLDevice dev = DLDevice{kDLCUDA, 0});
DLTensorUPtr makeDLTensor(DLDataType dtype, DLDevice dev, const std::vector<int64_t>& sizes,
                          const std::vector<int64_t>& strides, void* data);
DLConstTensorUPtr makeDLConstTensor(DLDataType dtype, DLDevice dev, const std::vector<int64_t>& sizes,
                                    const std::vector<int64_t>& strides, const void* data);

constexpr DLDataType kFloat32{kDLFloat, 32, 1};

}  // namespace tc
