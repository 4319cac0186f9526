// forwards to the op:: umbrella (reference: dali/array/op/unary.h)
#include "dali/array/op.h"
