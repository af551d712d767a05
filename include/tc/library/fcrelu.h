// tc/library/fcrelu.h of the reference: 1 fully-connected layer(s), each + bias and ReLU.
#pragma once

#include <string>

#include "tc/library/tc_text.h"

namespace tc {

constexpr static auto TC_FCRELU_NAME = "func_fcrelu";

inline const std::string TC_FCRELU = library_detail::fcreluChain(1, TC_FCRELU_NAME);

}  // namespace tc
