// forwards to the op:: umbrella (reference: dali/array/op/one_hot.h)
#include "dali/array/op.h"
