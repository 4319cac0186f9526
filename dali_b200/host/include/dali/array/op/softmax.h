// forwards to the op:: umbrella (reference: dali/array/op/softmax.h)
#include "dali/array/op.h"
