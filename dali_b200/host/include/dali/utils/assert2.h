// ASSERT2(condition, message): throws std::runtime_error(message) when the
// condition fails (reference: dali/utils/assert2.h:8-22, assert2.cpp).
#ifndef DALI_UTILS_ASSERT2_H
#define DALI_UTILS_ASSERT2_H

#include <stdexcept>
#include <string>

#include "dali/utils/make_message.h"

namespace utils {
inline void assert2(bool condition, const std::string& message) {
    if (!condition) throw std::runtime_error(message);
}
inline void assert2(bool condition) { assert2(condition, ""); }
}  // namespace utils

#define ASSERT2(condition, message) \
    if (!(condition)) utils::assert2(false, (message))

#define ASSERT2_SHAPE_ND(SHAPE, DIM, MSG) \
    if ((SHAPE).size() != (DIM))          \
        utils::assert2(false, utils::make_message(MSG, " was expecting dimension ", DIM, ", got shape ", SHAPE, "."));

#define ASSERT2_EQ(EXPECTED, ACTUAL, MSG) \
    if ((EXPECTED) != (ACTUAL))           \
        utils::assert2(false, utils::make_message("Expected ", EXPECTED, ", got ", ACTUAL, ": ", MSG, "."));

#endif
