// tc/library/group_convolution.h:23-45 of the reference: grouped valid 2-D convolution + bias.
#pragma once

#include <string>

#include "tc/core/check.h"
#include "tc/library/tc_text.h"

namespace tc {

constexpr static auto GROUP_CONVOLUTION2D_TC_NAME = "group_convolution";

inline std::string makeGroupConvolution2DTc(int strideH, int strideW) {
  TC_CHECK(strideH > 0 && strideW > 0) << "Stride must be greater than 0";
  return library_detail::conv2d(true, strideH, strideW);
}

}  // namespace tc
