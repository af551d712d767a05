// tc/library/3fcrelu.h of the reference: 3 fully-connected layer(s), each + bias and ReLU.
#pragma once

#include <string>

#include "tc/library/tc_text.h"

namespace tc {

constexpr static auto TC_3FCRELU_NAME = "func_3fcrelu";

inline const std::string TC_3FCRELU = library_detail::fcreluChain(3, TC_3FCRELU_NAME);

}  // namespace tc
