// tc/library/convolution.h:23-42 of the reference: valid 2-D convolution + bias, strides as literals.
#pragma once

#include <string>

#include "tc/core/check.h"
#include "tc/library/tc_text.h"

namespace tc {

constexpr static auto CONVOLUTION2D_TC_NAME = "convolution";

inline std::string makeConvolution2DTc(int strideH, int strideW) {
  TC_CHECK(strideH > 0 && strideW > 0) << "Stride must be greater than 0";
  return library_detail::conv2d(false, strideH, strideW);
}

}  // namespace tc
