// Seeding of the random operators (reference: dali/utils/random.h:36-41).  Every op::uniform /
// op::normal / op::bernoulli node draws one 31-bit seed from this process-wide mt19937 when it
// is built (the reference's GPU path draws utils::randinteger(0, 999999) per call,
// dali/array/op/random.cu.cpp:204-230); the numbers themselves come from a counter-based
// generator on the device.
#ifndef DALI_B200_UTILS_RANDOM_H
#define DALI_B200_UTILS_RANDOM_H

#include <random>

namespace utils {
int randint(int lower, int upper);
double randdouble(double lower = 0.0, double upper = 1.0);
namespace random {
void reseed();                 // from std::random_device
void set_seed(int new_seed);
std::mt19937& generator();
}  // namespace random
}  // namespace utils

#endif
