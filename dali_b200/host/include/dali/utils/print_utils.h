// Stream helpers used in error messages: utils::MS (a string built with <<)
// and operator<< for std::vector (reference: dali/utils/print_utils.h:17-37,
// print_utils.cpp; vectors print as "[a, b, c]").
#ifndef DALI_UTILS_PRINT_UTILS_H
#define DALI_UTILS_PRINT_UTILS_H

#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#define ELOG(EXP) std::cout << #EXP "\t=\t" << (EXP) << std::endl
#define SELOG(STR, EXP) std::cout << #STR "\t=\t" << (EXP) << std::endl

template <typename T>
std::ostream& operator<<(std::ostream& os, const std::vector<T>& values) {
    os << "[";
    for (size_t i = 0; i < values.size(); ++i) os << (i ? ", " : "") << values[i];
    return os << "]";
}

namespace utils {
class MS {
  public:
    std::stringstream stream;
    operator std::string() const { return stream.str(); }
    template <class T>
    MS& operator<<(const T& value) { stream << value; return *this; }
};

template <typename It>
std::string iter_to_str(It begin, It end) {
    std::stringstream out;
    for (bool first = true; begin != end; ++begin, first = false) out << (first ? "" : ", ") << *begin;
    return out.str();
}
}  // namespace utils

#endif
