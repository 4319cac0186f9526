// utils::make_message(args...): every argument streamed into one string
// (reference: dali/utils/make_message.h:6-22).
#ifndef DALI_UTILS_MAKE_MESSAGE_H
#define DALI_UTILS_MAKE_MESSAGE_H

#include <sstream>
#include <string>

#include "dali/utils/print_utils.h"   // operator<< for std::vector has to be visible to the template below

namespace utils {
template <typename... Args>
std::string make_message(const Args&... args) {
    std::ostringstream out;
    using expand = int[];
    (void)expand{0, ((void)(out << args), 0)...};
    return out.str();
}
}  // namespace utils

#endif
