// forwards to the op:: umbrella (reference: dali/array/op/random.h)
#include "dali/array/op.h"
