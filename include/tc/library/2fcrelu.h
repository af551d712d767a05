// tc/library/2fcrelu.h of the reference: 2 fully-connected layer(s), each + bias and ReLU.
#pragma once

#include <string>

#include "tc/library/tc_text.h"

namespace tc {

constexpr static auto TC_2FCRELU_NAME = "func_2fcrelu";

inline const std::string TC_2FCRELU = library_detail::fcreluChain(2, TC_2FCRELU_NAME);

}  // namespace tc
