// tc/library/4fcrelu.h of the reference: 4 fully-connected layer(s), each + bias and ReLU.
#pragma once

#include <string>

#include "tc/library/tc_text.h"

namespace tc {

constexpr static auto TC_4FCRELU_NAME = "func_4fcrelu";

inline const std::string TC_4FCRELU = library_detail::fcreluChain(4, TC_4FCRELU_NAME);

}  // namespace tc
